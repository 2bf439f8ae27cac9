/* SpMM for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference: the reference's SpMM
 * is a host loop over std::vector storage (src/core_ops.cpp:24-35) and knows
 * nothing about device memory.
 *
 * Who needs it.  The regular entry point, sp3_cuda_spmm_f32, takes its scratch
 * (partial rows of split long rows, arrival counters) from the caller, and the
 * Python front end gets that scratch from torch's allocator.  Some callers
 * cannot do either: code that runs while another component owns all device
 * memory (an inference server that hands out a fixed arena at start-up and
 * forbids later cudaMalloc because it would fragment or exceed the budget),
 * plug-ins and callbacks that run where an allocation could synchronise the
 * device or deadlock against a memory pool lock, and programs that talk to
 * this library through its C ABI alone, without torch.  For them
 * sp3_cuda_spmm_f32_noalloc computes exactly the same result but keeps its
 * scratch in a fixed array inside the library.  It calls no cudaMalloc, no
 * cudaFree and no allocating library routine.
 *
 * Cost and limit.  The array is SP3_NOALLOC_SCRATCH_BYTES (8 MiB) of device
 * memory on every GPU that loads the library, held until the process exits,
 * whether or not this function is ever called.  A call fits when
 *     nlong <= SP3_NOALLOC_MAX_SPLIT_ROWS   and
 *     SP3_NOALLOC_MAX_SPLIT_ROWS*4 + total_pieces * round_up(k, 4) * 4
 *         <= SP3_NOALLOC_SCRATCH_BYTES;
 * anything larger is refused with SP3_NOALLOC_E_TOO_LARGE and nothing is
 * launched.  (With k = 128 that is room for about 16,000 pieces of 512
 * nonzeros, i.e. 8 million nonzeros in split rows.)
 *
 * First call.  The first call on each device looks up the device address of
 * the array (cudaGetSymbolAddress) with that device current.  Make that first
 * call outside any CUDA stream capture.  First calls may come from several
 * host threads at once.  `stream` must be a stream of the device that is
 * current when the function is called (or 0): the array that is used is the
 * current device's.
 *
 * Sharing.  All calls on one device use the same array.  The counters are
 * cleared at the start of every call (a memset on the given stream), so stale
 * contents of an earlier call do no harm; but two calls that may run on the
 * GPU at the same time (different streams, no dependency between them) race
 * on the scratch and produce wrong rows.  Serialise them.
 *
 * Arguments: as sp3_cuda_spmm_f32 -- a CSR matrix (rowptr int64, colidx
 * int32, val), its work items (int32[nitems][4]) with the split-row tables
 * first_piece/npieces (int32[nlong]) as built by the framework's scheduler,
 * X [*, k] with leading dimension ldx, Y [nrows, k] with leading dimension
 * ldy, Y = beta*Y + A X.  All pointers are device pointers.  k, ldx and ldy
 * must be multiples of 4 and X, Y 16-byte aligned for the vector kernel;
 * otherwise the scalar kernel runs (it needs no scratch).
 * total_pieces = sum of npieces, piece_len = nonzeros per piece.
 *
 * Returns 0, a negative SP3_NOALLOC_E_* code, or a positive cudaError_t.
 */
#ifndef SP3_NOALLOC_H
#define SP3_NOALLOC_H

#define SP3_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)
#define SP3_NOALLOC_MAX_SPLIT_ROWS 16384
#define SP3_NOALLOC_E_ARG (-4)
#define SP3_NOALLOC_E_TOO_LARGE (-5)

#ifdef __cplusplus
extern "C" {
#endif

int sp3_cuda_spmm_f32_noalloc(int nrows, int nitems, const void* items, const long long* rowptr,
                              const int* colidx, const float* val, const float* X, long long ldx, int k,
                              float beta, float* Y, long long ldy, const int* first_piece, const int* npieces,
                              int nlong, int total_pieces, int piece_len, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SP3_NOALLOC_H */

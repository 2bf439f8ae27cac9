// Dense-panel SDDMM on the 5th-generation tensor cores (sm_100a, TF32).
//
// Where the nonzeros of a block of 128 consecutive local rows concentrate in a
// few columns (hub rows x hub columns of a power-law matrix), the block is
// cheaper as a small dense product than as a list of gathers: one CTA stages
// the 128 A rows and the N panel B rows in shared memory, a single thread
// issues `tcgen05.mma.cta_group::1.kind::tf32` over the k dimension with the
// 128 x N fp32 accumulator in tensor memory (TMEM), the tile is read back with
// `tcgen05.ld`, and only the positions that are nonzeros of S are kept:
//   out[pos] = sval * D[row_in_block][column_slot].
// The reference computes every nonzero with a scalar loop
// (src/core_ops.cpp:5-22); this path has no counterpart there.
//
// Operands are rounded to TF32 by the tensor core (10-bit mantissa), so the
// path is opt-in and tested with a matching tolerance.
//
// Shared-memory operand layout (K-major, no swizzle): 16-byte chunk c (4
// floats of k) of row r lives at byte (c * (ROWS + 1) + r) * 16.  A core
// matrix (8 rows x 16 B) is 128 contiguous bytes; the next 8 rows are SBO =
// 128 B away, the next k chunk LBO = (ROWS + 1) * 16 B away (the extra 16 B per
// chunk keep the staging stores of a warp, which writes one row = 32 chunks at
// a time, on distinct banks).  One MMA consumes 8 floats of k (two chunks).
// The accumulator tile is staged for sampling in the space of the A operand,
// which is dead once the MMAs have completed.
#include "sp3_cuda.cuh"

namespace sp3 {

constexpr int PANEL_M = 128;   // rows per panel (TMEM lanes)
constexpr int PANEL_N = 64;    // columns per panel (TMEM columns)
constexpr unsigned PANEL_WAIT_TRIES = 1u << 22;

// bytes of the A operand space: [k/4 chunks][129] float4, at least the 128 x 65 fp32 accumulator staging tile
__host__ __device__ inline size_t panel_a_bytes(int k) {
    const size_t a = (size_t)(k / 4) * (PANEL_M + 1) * 16, d = (size_t)PANEL_M * (PANEL_N + 1) * 4;
    return ((a > d ? a : d) + 127) / 128 * 128;
}

__device__ __forceinline__ unsigned p_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// K-major, SWIZZLE_NONE shared-memory matrix descriptor (version 1 = Blackwell).
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);        // start address, bits [0,14)
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;   // leading byte offset, bits [16,30)
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;   // stride byte offset, bits [32,46)
    d |= 1ull << 46;                                               // descriptor version, bits [46,48)
    return d;                                                      // base offset 0, layout type 0 (no swizzle)
}

// Instruction descriptor: D = F32, A = B = TF32, both K-major, M x N tile.
__host__ __device__ constexpr unsigned umma_idesc_tf32(int M, int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
}

__global__ void __launch_bounds__(128)
sddmm_panel_kernel(int npanels, const int* __restrict__ panel_row0, const int* __restrict__ panel_cols,
                   const int* __restrict__ panel_ptr, const unsigned char* __restrict__ e_row,
                   const unsigned char* __restrict__ e_col, const int* __restrict__ e_pos,
                   const float* __restrict__ e_sval, const float* __restrict__ A, long long lda, int nrows_a,
                   const float* __restrict__ B, long long ldb, int k, float* __restrict__ out, int* status) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int nchunk = k / 4;
    constexpr int LDA_S = PANEL_M + 1, LDB_S = PANEL_N + 1;                     // chunk strides in float4
    const size_t a_bytes = panel_a_bytes(k);
    float4* sA = reinterpret_cast<float4*>(smem);                               // [nchunk][129]
    float* sD = reinterpret_cast<float*>(smem);                                 // [128][65], reuses the A space
    float4* sB = reinterpret_cast<float4*>(smem + a_bytes);                     // [nchunk][65]
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(smem + a_bytes + (size_t)nchunk * LDB_S * 16);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bar + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned bar_addr = p_smem_u32(bar);

    if (tid == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_addr));
    if (warp == 0) {  // one warp allocates the accumulator columns and gives up the permit
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(p_smem_u32(tmem_slot)), "r"(PANEL_N));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = *tmem_slot;
    unsigned phase = 0;
    bool ok = true;

    for (int p = blockIdx.x; p < npanels && ok; p += gridDim.x) {
        const int r0 = panel_row0[p];
        // stage the 128 A rows and the 64 panel B rows: a warp reads one row per step, lane = 16-byte chunk
        // (coalesced), four rows in flight
        for (int rr = warp * 32; rr < warp * 32 + 32; rr += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int row = r0 + rr + u;
                const float4* src = reinterpret_cast<const float4*>(A + (long long)(row < nrows_a ? row : r0) * lda);
                v[u] = lane < nchunk ? __ldg(src + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (lane < nchunk) sA[(size_t)lane * LDA_S + rr + u] = v[u];
        }
        for (int rr = warp * 16; rr < warp * 16 + 16; rr += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4* src = reinterpret_cast<const float4*>(B + (long long)panel_cols[(size_t)p * PANEL_N + rr + u] * ldb);
                v[u] = lane < nchunk ? __ldg(src + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (lane < nchunk) sB[(size_t)lane * LDB_S + rr + u] = v[u];
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
        __syncthreads();
        if (tid == 0) {
            const unsigned a0 = p_smem_u32(sA), b0 = p_smem_u32(sB);
            const unsigned idesc = umma_idesc_tf32(PANEL_M, PANEL_N);
            for (int s = 0; s < k / 8; ++s) {  // 8 floats of k = two 16-byte chunks per MMA
                const unsigned long long da = umma_desc(a0 + (unsigned)s * 2u * LDA_S * 16u, LDA_S * 16u, 128u);
                const unsigned long long db = umma_desc(b0 + (unsigned)s * 2u * LDB_S * 16u, LDB_S * 16u, 128u);
                const unsigned acc = s > 0;
                asm volatile(
                    "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                    " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
                    :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
        }
        // bounded wait for the accumulator
        {
            unsigned done = 0;
            for (unsigned i = 0; i < PANEL_WAIT_TRIES && !done; ++i)
                asm volatile("{\n .reg .pred q;\n mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n selp.u32 %0, 1, 0, q;\n}\n"
                             : "=r"(done) : "r"(bar_addr), "r"(phase) : "memory");
            if (!done) { report(status, ST_WAIT_TIMEOUT, 300, p, 0); ok = false; }
            phase ^= 1;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            // warp w reads TMEM lanes 32w..32w+31 (= rows), 32 columns per load
#pragma unroll
            for (int c0 = 0; c0 < PANEL_N; c0 += 32) {
                unsigned v[32];
                const unsigned taddr = tmem_d + ((unsigned)(warp * 32) << 16) + (unsigned)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; ++j) sD[(size_t)tid * (PANEL_N + 1) + c0 + j] = __uint_as_float(v[j]);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (ok)
            for (int e = panel_ptr[p] + tid; e < panel_ptr[p + 1]; e += 128)
                out[e_pos[e]] = e_sval[e] * sD[(size_t)e_row[e] * (PANEL_N + 1) + e_col[e]];
        __syncthreads();  // sD, sA, sB are reused by the next panel
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(PANEL_N));
}

}  // namespace sp3

using namespace sp3;

// Panels: panel_row0[p] first local A row of the 128-row block, panel_cols[p*64 + j] the local B row of
// column slot j (unused slots: any valid row), entries panel_ptr[p]..panel_ptr[p+1] with (row in block,
// column slot, output position, S value).  k must be a multiple of 8 and at most 128.
// Returns 0, a cudaError_t, or -1 for an unsupported shape.
SP3_API int sp3_cuda_sddmm_panel_f32(int npanels, const int* panel_row0, const int* panel_cols, const int* panel_ptr,
                                     const unsigned char* e_row, const unsigned char* e_col, const int* e_pos,
                                     const float* e_sval, const float* A, long long lda, int nrows_a, const float* B,
                                     long long ldb, int k, float* out, int* status, void* stream) {
    if (npanels == 0) return 0;
    if (k % 8 || k < 8 || k > 128 || lda % 4 || ldb % 4 || (uintptr_t)A % 16 || (uintptr_t)B % 16) return -1;
    const size_t smem = panel_a_bytes(k) + (size_t)(k / 4) * (PANEL_N + 1) * 16 + 16;
    cudaError_t e = cudaFuncSetAttribute(sddmm_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(sddmm_panel_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int per_sm = 1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sddmm_panel_kernel, 128, smem);
    if (per_sm < 1) per_sm = 1;
    const int blocks = npanels < sms * per_sm ? npanels : sms * per_sm;
    sddmm_panel_kernel<<<blocks, 128, smem, (cudaStream_t)stream>>>(npanels, panel_row0, panel_cols, panel_ptr, e_row, e_col,
                                                                    e_pos, e_sval, A, lda, nrows_a, B, ldb, k, out, status);
    return (int)cudaGetLastError();
}

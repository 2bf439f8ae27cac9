// SDDMM with the column-side rows fetched by TMA gather (sm_100a, fp32).
//
// Same math and work decomposition as the local SDDMM kernel (local_ops.cu,
// reference loop src/core_ops.cpp:5-22), but the B rows of a batch of 32
// nonzeros are brought into shared memory by the tensor memory accelerator:
// eight `cp.async.bulk.tensor.2d ... tile::gather4` copies per batch, each
// naming four row indices of a 2-D tensor map over the local B block, complete
// on an mbarrier; the warp then reads the rows from shared memory.  Batches are
// multi-buffered per warp, so the copies of the next batch are in flight while
// a batch is reduced.  Every copy targets the shared memory of the issuing CTA only.
//
// Measured on B200 (R-MAT scale 20): this kernel is slower than the kernel that
// gathers with vector loads (k = 32: 0.35 vs 0.27 ms, k = 128: 2.6 vs 0.61 ms);
// a gather4 copy sustains roughly 10-20 bytes per clock per SM here against
// 40-60 for plain loads, so it is kept as an opt-in path (SP3_SDDMM_TMA=1).
//
// The tensor map describes [nrows x k] fp32 with a box of k x 1 elements; a
// gather4 copy therefore delivers 4 x k elements (4 rows) to consecutive
// shared memory.  The column coordinate of every copy is 0 (16-byte aligned).
#include "sp3_kernels.cuh"
#include "sp3_async.cuh"

#include <cuda.h>

namespace sp3 {

constexpr int TMA_MAX_STAGES = 8;
constexpr int TMA_ROWS = 32;            // B rows per batch and warp (one per lane)
__device__ __forceinline__ void tma_gather4(unsigned dst, const CUtensorMap* map, unsigned bar, int col, int r0,
                                            int r1, int r2, int r3) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        :: "r"(dst), "l"(map), "r"(bar), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}

template <int G, int R>
__global__ void __launch_bounds__(128)
sddmm_tma_kernel(const __grid_constant__ CUtensorMap mapB, long long nnz, const int* __restrict__ rowidx,
                 const int* __restrict__ colidx, const float* __restrict__ sval, const float* __restrict__ A,
                 long long lda, int nvec, float* __restrict__ out, int* status, int stages) {
    using V = float4;
    constexpr int SLOTS = 32 / G;
    constexpr int UU = 4 < G ? 4 : G;
    constexpr int NB = SDDMM_PER_SLOT / G;  // batches per work unit
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int slot = lane / G, gl = lane % G;
    const unsigned gmask = group_mask<G>(slot);
    const unsigned row_bytes = (unsigned)nvec * 16u;
    const unsigned stage_bytes = TMA_ROWS * row_bytes;
    // layout: [warps][stages][32 rows][k floats] then the mbarriers [warps][stages]
    unsigned char* my_rows = smem_raw + (size_t)wid * stages * stage_bytes;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + (size_t)nw * stages * stage_bytes);
    const unsigned bar0 = smem_u32(bars + wid * stages);
    if (lane == 0)
        for (int s = 0; s < stages; ++s) mbar_init(bar0 + 8u * s, 1);
    mbar_init_fence();
    __syncthreads();

    const V* Av = reinterpret_cast<const V*>(A);
    const long long lda_v = lda / 4;
    const long long warp0 = (long long)blockIdx.x * nw + wid;
    const long long nwarps = (long long)gridDim.x * nw;
    const long long per_unit = (long long)SLOTS * SDDMM_PER_SLOT;
    const long long n_units = (nnz + per_unit - 1) / per_unit;
    const long long my_units = warp0 < n_units ? (n_units - warp0 + nwarps - 1) / nwarps : 0;
    const long long total_q = my_units * NB;  // this warp's batches, in order

    // position of this lane's nonzero in batch q of this warp
    auto lane_pos = [&](long long q) -> long long {
        const long long unit = warp0 + (q / NB) * nwarps;
        return (unit * SLOTS + slot) * (long long)SDDMM_PER_SLOT + (q % NB) * G + gl;
    };
    // issue the 8 gather4 copies of batch q: lane L's nonzero gets shared-memory row L of the stage
    auto issue = [&](long long q) {
        const int st = (int)(q % stages);
        const long long i = lane_pos(q);
        const int my_c = i < nnz ? __ldg(colidx + i) : 0;
        const int c1 = __shfl_down_sync(0xffffffffu, my_c, 1);
        const int c2 = __shfl_down_sync(0xffffffffu, my_c, 2);
        const int c3 = __shfl_down_sync(0xffffffffu, my_c, 3);
        const unsigned bar = bar0 + 8u * st;
        if (lane == 0) mbar_expect_tx(bar, stage_bytes);
        __syncwarp();
        if ((lane & 3) == 0)
            tma_gather4(smem_u32(my_rows + (size_t)st * stage_bytes + (size_t)lane * row_bytes), &mapB, bar, 0, my_c, c1,
                        c2, c3);
    };

    for (long long q = 0; q < stages - 1 && q < total_q; ++q) issue(q);
    int cur_row = -1;
    V a[R];
#pragma unroll
    for (int r = 0; r < R; ++r) a[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long q = 0; q < total_q; ++q) {
        // the stage refilled here was read in the previous iteration, which ended with __syncwarp()
        if (q + stages - 1 < total_q) issue(q + stages - 1);
        const int st = (int)(q % stages);
        if (!mbar_wait(bar0 + 8u * st, (unsigned)((q / stages) & 1))) {
            report(status, ST_WAIT_TIMEOUT, 200, (int)blockIdx.x, st);
            break;
        }
        if (q % NB == 0) cur_row = -1;
        const long long my_i = lane_pos(q);
        const bool valid = my_i < nnz;
        const int my_r = valid ? __ldg(rowidx + my_i) : -1;
        const V* rows = reinterpret_cast<const V*>(my_rows + (size_t)st * stage_bytes);
        float my_out = 0.f;
#pragma unroll
        for (int j = 0; j < G; j += UU) {
            int rr[UU];
            float acc[UU];
#pragma unroll
            for (int u = 0; u < UU; ++u) rr[u] = __shfl_sync(gmask, my_r, j + u, G);
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                if (rr[u] >= 0 && rr[u] != cur_row) {
                    cur_row = rr[u];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const int v = gl + r * G;
                        a[r] = v < nvec ? __ldg(Av + (long long)cur_row * lda_v + v) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                const V* brow = rows + (size_t)(slot * G + j + u) * nvec;
                float d = 0.f;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int v = gl + r * G;
                    if (v < nvec) d += vdot(a[r], brow[v]);
                }
                acc[u] = rr[u] >= 0 ? d : 0.f;
            }
            group_transpose_reduce<float, G, UU>(acc, gmask, gl);
            const float mine = __shfl_sync(gmask, acc[0], (gl % UU) * (G / UU), G);
            if (gl / UU == j / UU) my_out = mine;
        }
        if (valid) out[my_i] = sval ? my_out * __ldg(sval + my_i) : my_out;
        __syncwarp();  // every lane is done with this stage before it is refilled
    }
}

// ---------------------------------------------------------------------------
// SpMM twin: the X rows of a batch of 32 nonzeros arrive by eight gather4 copies; the warp then walks the batch
// in order, lane = 16-byte vector of the row (two per lane for k = 256), and adds val * X row into the running
// sum of the current output row.  A warp owns units of 256 consecutive nonzeros of the row-sorted stream; rows
// that lie wholly inside a unit are updated with plain loads and stores, the first and the last row of a unit may
// continue in a neighbouring unit and are added with 16-byte vector atomics.  Y must hold beta * Y before the
// kernel (spmm_scale_kernel); sums of rows that span three or more units depend on the order of the atomics.
// Reference loop: src/core_ops.cpp:24-35.
// ---------------------------------------------------------------------------
constexpr int SPMM_TMA_NB = 8;  // batches of 32 nonzeros per unit

__global__ void spmm_scale_kernel(float* __restrict__ Y, long long ldy, long long nrows, int nvec, float beta) {
    const long long total = nrows * nvec;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        float4* y = reinterpret_cast<float4*>(Y + (e / nvec) * ldy) + e % nvec;
        *y = beta != 0.f ? vscale(beta, *y) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

__global__ void __launch_bounds__(128)
spmm_tma_kernel(const __grid_constant__ CUtensorMap mapX, long long nnz, const int* __restrict__ rowidx,
                const int* __restrict__ colidx, const float* __restrict__ val, int nvec, float* __restrict__ Y,
                long long ldy, int* status, int stages) {
    using V = float4;
    constexpr int NB = SPMM_TMA_NB;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const unsigned row_bytes = (unsigned)nvec * 16u;
    const unsigned stage_bytes = TMA_ROWS * row_bytes;
    unsigned char* my_rows = smem_raw + (size_t)wid * stages * stage_bytes;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + (size_t)nw * stages * stage_bytes);
    const unsigned bar0 = smem_u32(bars + wid * stages);
    if (lane == 0)
        for (int s = 0; s < stages; ++s) mbar_init(bar0 + 8u * s, 1);
    mbar_init_fence();
    __syncthreads();

    const long long warp0 = (long long)blockIdx.x * nw + wid;
    const long long nwarps = (long long)gridDim.x * nw;
    const long long per_unit = (long long)NB * TMA_ROWS;
    const long long n_units = (nnz + per_unit - 1) / per_unit;
    const long long my_units = warp0 < n_units ? (n_units - warp0 + nwarps - 1) / nwarps : 0;
    const long long total_q = my_units * NB;
    auto unit_begin = [&](long long q) -> long long { return (warp0 + (q / NB) * nwarps) * per_unit; };
    auto lane_pos = [&](long long q) -> long long { return unit_begin(q) + (q % NB) * TMA_ROWS + lane; };
    auto issue = [&](long long q) {
        const int st = (int)(q % stages);
        const long long i = lane_pos(q);
        const int my_c = i < nnz ? __ldg(colidx + i) : 0;
        const int c1 = __shfl_down_sync(0xffffffffu, my_c, 1);
        const int c2 = __shfl_down_sync(0xffffffffu, my_c, 2);
        const int c3 = __shfl_down_sync(0xffffffffu, my_c, 3);
        const unsigned bar = bar0 + 8u * st;
        if (lane == 0) mbar_expect_tx(bar, stage_bytes);
        __syncwarp();
        if ((lane & 3) == 0)
            tma_gather4(smem_u32(my_rows + (size_t)st * stage_bytes + (size_t)lane * row_bytes), &mapX, bar, 0, my_c, c1,
                        c2, c3);
    };

    const long long ldy_v = ldy / 4;
    V* Yv = reinterpret_cast<V*>(Y);
    int cur_row = -1, first_row = -1, last_row = -1;
    V acc[2];
    acc[0] = acc[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    auto flush = [&]() {
        if (cur_row < 0) return;
        const bool shared_row = cur_row == first_row || cur_row == last_row;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int v = lane + 32 * r;
            if (v < nvec) {
                V* y = Yv + (long long)cur_row * ldy_v + v;
                if (shared_row) atomicAdd(y, acc[r]);
                else { V o = *y; vadd(o, acc[r]); *y = o; }
            }
            acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        cur_row = -1;
    };

    for (long long q = 0; q < stages - 1 && q < total_q; ++q) issue(q);
    for (long long q = 0; q < total_q; ++q) {
        if (q + stages - 1 < total_q) issue(q + stages - 1);
        const int st = (int)(q % stages);
        if (!mbar_wait(bar0 + 8u * st, (unsigned)((q / stages) & 1))) {
            report(status, ST_WAIT_TIMEOUT, 201, (int)blockIdx.x, st);
            break;
        }
        if (q % NB == 0) {
            const long long b = unit_begin(q);
            const long long e = b + per_unit < nnz ? b + per_unit : nnz;
            first_row = __ldg(rowidx + b);
            last_row = __ldg(rowidx + e - 1);
        }
        const long long my_i = lane_pos(q);
        const bool valid = my_i < nnz;
        const int my_r = valid ? __ldg(rowidx + my_i) : -1;
        const float my_v = valid ? __ldg(val + my_i) : 0.f;
        const V* rows = reinterpret_cast<const V*>(my_rows + (size_t)st * stage_bytes);
        for (int j = 0; j < TMA_ROWS; ++j) {
            const int rj = __shfl_sync(0xffffffffu, my_r, j);
            const float vj = __shfl_sync(0xffffffffu, my_v, j);
            if (rj < 0) break;  // uniform: past the end of the stream
            if (rj != cur_row) { flush(); cur_row = rj; }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int v = lane + 32 * r;
                if (v < nvec) vfma(acc[r], vj, rows[(size_t)j * nvec + v]);
            }
        }
        if (q % NB == NB - 1) flush();
        __syncwarp();  // every lane is done with this stage before it is refilled
    }
    flush();
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

}  // namespace sp3

using namespace sp3;

// Returns 0, a cudaError_t (> 0), or a negative code: -1 unsupported shape
// (k not a multiple of 8, k > 256, misaligned B / ldb), -2 tensor map encoding
// failed or is not available.
SP3_API int sp3_cuda_sddmm_tma_f32(long long nnz, const int* ri, const int* ci, const float* sv, const float* A,
                                   long long lda, const float* B, long long ldb, long long nrows_b, int k,
                                   float* out, int* status, void* stream) {
    if (nnz == 0) return 0;
    // k a multiple of 8: a gather4 copy lands 4 rows = 16 * k bytes at a 128-byte aligned shared-memory address
    if (k % 8 || k > 256 || k < 8 || lda % 4 || ldb % 4 || (uintptr_t)A % 16 || (uintptr_t)B % 16 || nrows_b <= 0) return -1;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return -2;
    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)nrows_b};
    const cuuint64_t gstride[1] = {(cuuint64_t)ldb * 4};
    const cuuint32_t box[2] = {(cuuint32_t)k, 1};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)B, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return -2;
    const int nvec = k / 4;
    // Two stages per warp by default: measured on B200, more resident warps (several CTAs per SM) beat a
    // deeper ring per warp (R-MAT scale 20, k = 32: 0.35 ms with 2 stages, 1.6 ms with 8).
    static const int want_warps = env_int("SP3_TMA_WARPS", 4);
    static const int want_stages = env_int("SP3_TMA_STAGES", 2);
    const size_t stage_bytes = (size_t)TMA_ROWS * k * 4;
    int warps = want_warps < 1 ? 1 : (want_warps > 4 ? 4 : want_warps);
    while (warps > 1 && (200 * 1024) / (warps * stage_bytes) < 2) --warps;
    int stages = (int)((200 * 1024) / (warps * stage_bytes));
    if (stages > want_stages) stages = want_stages;
    if (stages > TMA_MAX_STAGES) stages = TMA_MAX_STAGES;
    if (stages < 2) return -1;
    const size_t smem = stage_bytes * stages * warps + (size_t)warps * stages * 8;
    int G, R;
    pick_shape(nvec, &G, &R, false);
    cudaStream_t st = (cudaStream_t)stream;
    const long long per_unit = (long long)(32 / G) * SDDMM_PER_SLOT;
    const long long units = (nnz + per_unit - 1) / per_unit;
    const long long needed = (units + warps - 1) / warps;
#define SP3_TMA(GG, RR)                                                                                          \
    {                                                                                                            \
        cudaError_t e = cudaFuncSetAttribute(sddmm_tma_kernel<GG, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             (int)smem);                                                         \
        if (e != cudaSuccess) return (int)e;                                                                     \
        sddmm_tma_kernel<GG, RR><<<persistent_blocks(sddmm_tma_kernel<GG, RR>, needed, 32 * warps, smem),         \
                                   32 * warps, smem, st>>>(map, nnz, ri, ci, sv, A, lda, nvec, out, status, stages); \
    }
    if (R == 2) {
        switch (G) { case 1: SP3_TMA(1, 2) break; case 2: SP3_TMA(2, 2) break; case 4: SP3_TMA(4, 2) break;
                     case 8: SP3_TMA(8, 2) break; default: SP3_TMA(16, 2) break; }
    } else if (R == 4) {
        SP3_TMA(16, 4)
    } else return -1;
#undef SP3_TMA
    return (int)cudaGetLastError();
}

// Y = beta * Y + S * X for a row-sorted COO stream (rowidx ascending).  Returns 0, a cudaError_t (> 0), -1 for an
// unsupported shape (k not a multiple of 8, k > 256, misaligned X / Y), -2 when no tensor map can be encoded.
SP3_API int sp3_cuda_spmm_tma_f32(long long nnz, const int* ri, const int* ci, const float* sv, const float* X,
                                  long long ldx, long long nrows_x, int k, float beta, float* Y, long long ldy,
                                  long long nrows_y, int* status, void* stream) {
    // k a multiple of 8: a gather4 copy lands 4 rows = 16 * k bytes at a 128-byte aligned shared-memory address
    if (k % 8 || k > 256 || k < 8 || ldx % 4 || ldy % 4 || (uintptr_t)X % 16 || (uintptr_t)Y % 16 || nrows_x <= 0) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    const int nvec = k / 4;
    if (nrows_y > 0) {
        const long long total = nrows_y * nvec;
        const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
        spmm_scale_kernel<<<blocks, 256, 0, st>>>(Y, ldy, nrows_y, nvec, beta);
    }
    if (nnz == 0) return (int)cudaGetLastError();
    EncodeTiledFn enc = encode_fn();
    if (!enc) return -2;
    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)nrows_x};
    const cuuint64_t gstride[1] = {(cuuint64_t)ldx * 4};
    const cuuint32_t box[2] = {(cuuint32_t)k, 1};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)X, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return -2;
    const size_t stage_bytes = (size_t)TMA_ROWS * k * 4;
    int warps = 4;
    while (warps > 1 && (200 * 1024) / (warps * stage_bytes) < 2) --warps;
    const int stages = 2;
    const size_t smem = stage_bytes * stages * warps + (size_t)warps * stages * 8;
    cudaError_t e = cudaFuncSetAttribute(spmm_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const long long per_unit = (long long)SPMM_TMA_NB * TMA_ROWS;
    const long long units = (nnz + per_unit - 1) / per_unit;
    const long long needed = (units + warps - 1) / warps;
    spmm_tma_kernel<<<persistent_blocks(spmm_tma_kernel, needed, 32 * warps, smem), 32 * warps, smem, st>>>(
        map, nnz, ri, ci, sv, nvec, Y, ldy, status, stages);
    return (int)cudaGetLastError();
}

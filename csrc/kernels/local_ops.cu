// Local (one GPU, no communication) kernels for sm_100a:
//   SDDMM over a row-sorted nonzero list, SpMM over scheduled work items,
//   row gather / scatter / scatter-add, operand fill, checksum, index remaps.
//
// They replace the scalar CPU loops of the reference: sddmm / spmm
// src/core_ops.cpp:5-35, pack / unpack / sum src/comm.hpp:90-103,166-189,
// ReMapIndices src/SparseMatrix.hpp:100-106, checksum
// miniapp/bench_spmm.cpp:117.
//
// Layout of the math: a dense row of k elements is spread over a group of G
// lanes (G = power of two <= 32), each lane holding R 16-byte vectors, so one
// warp works on 32/G nonzeros (SDDMM) or rows (SpMM) at a time and every
// global access is a full-width vector load of a contiguous row segment.
// Both kernels are bound by the gathers of dense rows from HBM/L2; the
// unroll factor U keeps U independent row loads in flight per lane.
#include "sp3_kernels.cuh"

#include <cstdlib>

namespace sp3 {

// ---------------------------------------------------------------------------
// SDDMM: out[i] = sval[i] * <A[rowidx[i]], B[colidx[i]]>; persistent grid,
// warps stride over work units (see sddmm_warp_unit).
// ---------------------------------------------------------------------------
template <typename T, int G, int R, int U>
__global__ void __launch_bounds__(256, sddmm_min_blocks(R))
sddmm_vec_kernel(long long nnz, const int* __restrict__ rowidx, const int* __restrict__ colidx,
                 const T* __restrict__ sval, const T* __restrict__ A, long long lda,
                 const T* __restrict__ B, long long ldb, int nvec, T* __restrict__ out, const int* __restrict__ orig) {
    using V = typename Vec<T>::type;
    constexpr int SLOTS = 32 / G;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    const RowsByStride<T> arows{reinterpret_cast<const V*>(A), lda / Vec<T>::N};
    const StoreLocal<T> store{out, sval, orig};
    for (long long unit = warp0; unit * SLOTS * (long long)SDDMM_PER_SLOT < nnz; unit += nwarps)
        sddmm_warp_unit<T, G, R, U>(unit, nnz, rowidx, colidx, arows, reinterpret_cast<const V*>(B),
                                    ldb / Vec<T>::N, nvec, store, lane);
}

// Any k, any leading dimension: one warp per nonzero slot, scalar loads.
template <typename T>
__global__ void __launch_bounds__(256)
sddmm_scalar_kernel(long long nnz, const int* __restrict__ rowidx, const int* __restrict__ colidx,
                    const T* __restrict__ sval, const T* __restrict__ A, long long lda,
                    const T* __restrict__ B, long long ldb, int k, T* __restrict__ out) {
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long i = warp; i < nnz; i += nwarps) {
        const T* a = A + (long long)rowidx[i] * lda;
        const T* b = B + (long long)colidx[i] * ldb;
        T acc = 0;
        for (int j = lane; j < k; j += 32) acc += a[j] * b[j];
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
        if (lane == 0) out[i] = sval ? acc * sval[i] : acc;
    }
}

// ---------------------------------------------------------------------------
// SpMM over work items (see spmm_warp_item): Y[row] = beta * Y[row] + sum.
// Rows without nonzeros are covered by rows items, so beta is applied to
// every row exactly once.
// ---------------------------------------------------------------------------
#ifndef SP3_SPMM_ITEMS_PER_STEP
#define SP3_SPMM_ITEMS_PER_STEP 4
#endif
constexpr int SPMM_ITEMS_PER_STEP = SP3_SPMM_ITEMS_PER_STEP;

template <typename T, int G, int R, int U>
__global__ void __launch_bounds__(256)
spmm_items_kernel(int nitems, const int4* __restrict__ items, const long long* __restrict__ rowptr,
                  const int* __restrict__ colidx, const T* __restrict__ val, const T* __restrict__ X,
                  long long ldx, int nvec, T beta, T* __restrict__ Y, long long ldy, SpmmLong lg) {
    using V = typename Vec<T>::type;
    const int warp0 = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const int nwarps = (int)(((long long)gridDim.x * blockDim.x) >> 5);
    const int lane = threadIdx.x & 31;
    const EmitLocal<T> emit{reinterpret_cast<V*>(Y), ldy / Vec<T>::N, beta};
    if (lg.ticket) {
        // dynamic hand-out, SPMM_ITEMS_PER_STEP items per ticket: rows of a power-law matrix differ too much in
        // cost for a fixed assignment to balance
        const int step = per_ticket(nitems, nwarps, SPMM_ITEMS_PER_STEP);
        for (;;) {
            int base = 0;
            if (lane == 0) base = atomicAdd(lg.ticket, step);
            base = __shfl_sync(0xffffffffu, base, 0);
            if (base >= nitems) break;
            for (int it = base; it < base + step && it < nitems; ++it)
                spmm_warp_item<T, G, R, U>(__ldg(items + it), rowptr, colidx, val, reinterpret_cast<const V*>(X),
                                           ldx / Vec<T>::N, nvec, emit, lg, lane);
        }
        return;
    }
    for (int it = warp0; it < nitems; it += nwarps)
        spmm_warp_item<T, G, R, U>(__ldg(items + it), rowptr, colidx, val, reinterpret_cast<const V*>(X),
                                   ldx / Vec<T>::N, nvec, emit, lg, lane);
}

// Any k / leading dimension: one warp per row, scalar loads, no schedule.
template <typename T>
__global__ void __launch_bounds__(256)
spmm_scalar_kernel(int nrows, const long long* __restrict__ rowptr, const int* __restrict__ colidx,
                   const T* __restrict__ val, const T* __restrict__ X, long long ldx, int k, T beta,
                   T* __restrict__ Y, long long ldy) {
    const int warp = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (warp >= nrows) return;
    for (int j = lane; j < k; j += 32) {
        T acc = 0;
        for (long long p = rowptr[warp]; p < rowptr[warp + 1]; ++p) acc += val[p] * X[(long long)colidx[p] * ldx + j];
        T* y = Y + (long long)warp * ldy + j;
        *y = beta != (T)0 ? beta * *y + acc : acc;
    }
}

// ---------------------------------------------------------------------------
// rows: mode 0 dst[i] = src[idx[i]]; 1 dst[idx[i]] = src[i]; 2 dst[idx[i]] += src[i]
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
rows_kernel(int mode, long long n, const long long* __restrict__ idx, const T* __restrict__ src, long long lds,
            T* __restrict__ dst, long long ldd, int k) {
    using V = typename Vec<T>::type;
    const int nvec = VEC ? k / Vec<T>::N : k;
    const int G = pick_group(nvec);
    const int lane = threadIdx.x & 31, slot = lane / G, gl = lane % G;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long i = warp * (32 / G) + slot;
    if (i >= n) return;
    const long long j = idx[i];
    const long long srow = mode == 0 ? j : i, drow = mode == 0 ? i : j;
    if (VEC) {
        const V* s = reinterpret_cast<const V*>(src + srow * lds);
        V* d = reinterpret_cast<V*>(dst + drow * ldd);
        for (int v = gl; v < nvec; v += G) {
            V x = __ldg(s + v);
            if (mode == 2) { V o = d[v]; vadd(o, x); d[v] = o; }
            else d[v] = x;
        }
    } else {
        const T* s = src + srow * lds;
        T* d = dst + drow * ldd;
        for (int v = gl; v < nvec; v += G) {
            if (mode == 2) d[v] += s[v];
            else d[v] = s[v];
        }
    }
}

// ---------------------------------------------------------------------------
// Operand fill: the device twin of sp3_fill_rows_* (csrc/host/generate.cpp).
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ unsigned long long rnd(unsigned long long seed, unsigned long long stream,
                                                  unsigned long long idx) {
    return mix64(mix64(seed ^ (stream * 0xD6E8FEB86659FD93ull)) + idx * 0x9E3779B97F4A7C15ull);
}
__device__ __forceinline__ double u01(unsigned long long bits) {
    return (double)(bits >> 11) * (1.0 / 9007199254740992.0);
}

template <typename T>
__global__ void fill_rows_kernel(const long long* __restrict__ gid, long long nrows, long long col0, int ncols,
                                 long long ld, long long kglobal, int kind, double cval,
                                 unsigned long long seed, unsigned long long stream, T* __restrict__ out) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nrows * ncols) return;
    const long long i = t / ncols;
    const int j = (int)(t % ncols);
    double v;
    if (kind == 0) {
        const unsigned long long e = (unsigned long long)gid[i] * (unsigned long long)kglobal + col0 + j;
        double u1 = u01(rnd(seed, stream, 2 * e)), u2 = u01(rnd(seed, stream, 2 * e + 1));
        if (u1 < 1e-300) u1 = 1e-300;
        v = sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
    } else if (kind == 1) v = (double)gid[i] / 1000.0;
    else v = cval;
    out[i * ld + j] = (T)v;
}

// ---------------------------------------------------------------------------
// checksum: fixed-shape two-stage sum in fp64 (bitwise reproducible).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) sum_stage1(const T* __restrict__ x, long long n, double* __restrict__ part) {
    __shared__ double sh[256];
    double acc = 0;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256) acc += (double)x[i];
    sh[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) { if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s]; __syncthreads(); }
    if (threadIdx.x == 0) part[blockIdx.x] = sh[0];
}
__global__ void __launch_bounds__(256) sum_stage2(const double* __restrict__ part, int n, double* __restrict__ out) {
    __shared__ double sh[256];
    double acc = 0;
    for (int i = threadIdx.x; i < n; i += 256) acc += part[i];
    sh[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) { if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s]; __syncthreads(); }
    if (threadIdx.x == 0) out[0] = sh[0];
}

// ---------------------------------------------------------------------------
// index utilities (setup time): out[i] = table[idx[i]], inv[perm[i]] = i,
// touch masks with atomicOr.
// ---------------------------------------------------------------------------
__global__ void remap_kernel(long long n, const int* __restrict__ idx, const int* __restrict__ table,
                             long long table_len, int* __restrict__ out, int* status) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int j = idx[i];
    if (j < 0 || j >= table_len) { report(status, ST_BAD_INDEX, 0, (int)i, j); out[i] = -1; return; }
    out[i] = table[j];
}
__global__ void invert_perm_kernel(long long n, const long long* __restrict__ perm, long long* __restrict__ inv,
                                   int* status) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long j = perm[i];
    if (j < 0 || j >= n) { report(status, ST_BAD_INDEX, 1, (int)i, (int)j); return; }
    inv[j] = i;
}
__global__ void touch_masks_kernel(long long nnz, const int* __restrict__ rows, const int* __restrict__ cols,
                                   const int* __restrict__ rowmap, const int* __restrict__ colmap,
                                   unsigned long long* __restrict__ row_mask, unsigned long long* __restrict__ col_mask) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    const int r = rows[i], c = cols[i];
    atomicOr(row_mask + r, 1ull << colmap[c]);
    atomicOr(col_mask + c, 1ull << rowmap[r]);
}

// Debug check: every idx[i] lies in [0, limit); the first offender is recorded in the status words
// {ST_BAD_INDEX, which, position, value} and nothing else happens (no trap).
__global__ void check_range_kernel(long long n, const int* __restrict__ idx, int limit, int which, int* status) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int v = idx[i];
    if (v < 0 || v >= limit) report(status, ST_BAD_INDEX, which, (int)i, v);
}

// ---- dispatch ---------------------------------------------------------------
template <typename T>
int launch_sddmm(long long nnz, const int* ri, const int* ci, const T* sv, const T* A, long long lda, const T* B,
                 long long ldb, int k, T* out, cudaStream_t st, const int* orig = nullptr) {
    if (nnz == 0) return 0;
    constexpr int VN = Vec<T>::N;
    const bool vec_ok = k % VN == 0 && lda % VN == 0 && ldb % VN == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)B % 16 == 0;
    const int nvec = k / VN;
    if (!vec_ok || nvec > 256) {
        if (orig) return -1;  // the scatter form exists for the vector kernel only
        long long warps = nnz < (1ll << 22) ? nnz : (1ll << 22);
        sddmm_scalar_kernel<T><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(nnz, ri, ci, sv, A, lda, B, ldb, k, out);
        return (int)cudaGetLastError();
    }
    int G, R;
    pick_shape(nvec, &G, &R, false);
    const long long slots = (nnz + SDDMM_PER_SLOT - 1) / SDDMM_PER_SLOT;
    const long long warps = (slots + (32 / G) - 1) / (32 / G);
    const long long needed = (warps + 7) / 8;
#define SP3_SDDMM(GG, RR)                                                                                      \
    sddmm_vec_kernel<T, GG, RR, (RR >= 8 ? 2 : 4)>                                                             \
        <<<persistent_blocks(sddmm_vec_kernel<T, GG, RR, (RR >= 8 ? 2 : 4)>, needed), 256, 0, st>>>(           \
            nnz, ri, ci, sv, A, lda, B, ldb, nvec, out, orig)
    SP3_DISPATCH_GR(SP3_SDDMM)
#undef SP3_SDDMM
    return (int)cudaGetLastError();
}

template <typename T>
int launch_spmm(int nrows, int nitems, const int4* items, const long long* rowptr, const int* ci, const T* val,
                const T* X, long long ldx, int k, T beta, T* Y, long long ldy, SpmmLong lg, cudaStream_t st) {
    if (nrows == 0) return 0;
    constexpr int VN = Vec<T>::N;
    const bool vec_ok = k % VN == 0 && ldx % VN == 0 && ldy % VN == 0 && (uintptr_t)X % 16 == 0 &&
                        (uintptr_t)Y % 16 == 0 && items != nullptr && (lg.ldc % VN == 0);
    const int nvec = k / VN;
    if (!vec_ok || nvec > 256) {
        spmm_scalar_kernel<T><<<(unsigned)(((long long)nrows * 32 + 255) / 256), 256, 0, st>>>(nrows, rowptr, ci, val, X, ldx, k, beta, Y, ldy);
        return (int)cudaGetLastError();
    }
    int G, R;
    pick_shape(nvec, &G, &R, true);
    if (lg.ticket) {
        cudaError_t e = cudaMemsetAsync(lg.ticket, 0, sizeof(int), st);
        if (e != cudaSuccess) return (int)e;
    }
    const long long needed = ((long long)nitems + 7) / 8;
#define SP3_SPMM(GG, RR)                                                                                       \
    spmm_items_kernel<T, GG, RR, (RR >= 8 ? 2 : 4)>                                                            \
        <<<persistent_blocks(spmm_items_kernel<T, GG, RR, (RR >= 8 ? 2 : 4)>, needed), 256, 0, st>>>(          \
            nitems, items, rowptr, ci, val, X, ldx, nvec, beta, Y, ldy, lg)
    SP3_DISPATCH_GR(SP3_SPMM)
#undef SP3_SPMM
    return (int)cudaGetLastError();
}

template <typename T>
int launch_rows(int mode, long long n, const long long* idx, const T* src, long long lds, T* dst, long long ldd, int k,
                cudaStream_t st) {
    if (n == 0) return 0;
    constexpr int VN = Vec<T>::N;
    const bool vec_ok = k % VN == 0 && lds % VN == 0 && ldd % VN == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)dst % 16 == 0;
    const int nvec = vec_ok ? k / VN : k;
    const int per_warp = 32 / pick_group(nvec);
    const long long warps = (n + per_warp - 1) / per_warp;
    const unsigned blocks = (unsigned)((warps + 7) / 8);
    if (vec_ok) rows_kernel<T, true><<<blocks, 256, 0, st>>>(mode, n, idx, src, lds, dst, ldd, k);
    else rows_kernel<T, false><<<blocks, 256, 0, st>>>(mode, n, idx, src, lds, dst, ldd, k);
    return (int)cudaGetLastError();
}

}  // namespace sp3

using namespace sp3;

SP3_API int sp3_cuda_sddmm_f32(long long nnz, const int* ri, const int* ci, const float* sv, const float* A,
                               long long lda, const float* B, long long ldb, int k, float* out, void* stream) {
    return launch_sddmm<float>(nnz, ri, ci, sv, A, lda, B, ldb, k, out, (cudaStream_t)stream);
}
// out[orig[i]] = sval[i] * <A[ri[i]], B[ci[i]]>: SDDMM over a subset of the nonzeros, results scattered to their
// positions in the full value array (used next to the dense-panel kernel).
SP3_API int sp3_cuda_sddmm_orig_f32(long long nnz, const int* ri, const int* ci, const float* sv, const float* A,
                                    long long lda, const float* B, long long ldb, int k, float* out, const int* orig,
                                    void* stream) {
    return launch_sddmm<float>(nnz, ri, ci, sv, A, lda, B, ldb, k, out, (cudaStream_t)stream, orig);
}
SP3_API int sp3_cuda_sddmm_f64(long long nnz, const int* ri, const int* ci, const double* sv, const double* A,
                               long long lda, const double* B, long long ldb, int k, double* out, void* stream) {
    return launch_sddmm<double>(nnz, ri, ci, sv, A, lda, B, ldb, k, out, (cudaStream_t)stream);
}

// items may be null (then the unscheduled one-warp-per-row kernel runs).
// Long-row arguments may be null/0 when the schedule has no long rows.
SP3_API int sp3_cuda_spmm_f32(int nrows, int nitems, const void* items, const long long* rowptr, const int* ci,
                              const float* val, const float* X, long long ldx, int k, float beta, float* Y,
                              long long ldy, const int* first_piece, const int* npieces, int* counters,
                              void* carry, long long ldc, int piece_len, int* ticket, void* stream) {
    SpmmLong lg{first_piece, npieces, counters, carry, ldc, piece_len, ticket};
    return launch_spmm<float>(nrows, nitems, (const int4*)items, rowptr, ci, val, X, ldx, k, beta, Y, ldy, lg,
                              (cudaStream_t)stream);
}
SP3_API int sp3_cuda_spmm_f64(int nrows, int nitems, const void* items, const long long* rowptr, const int* ci,
                              const double* val, const double* X, long long ldx, int k, double beta, double* Y,
                              long long ldy, const int* first_piece, const int* npieces, int* counters,
                              void* carry, long long ldc, int piece_len, int* ticket, void* stream) {
    SpmmLong lg{first_piece, npieces, counters, carry, ldc, piece_len, ticket};
    return launch_spmm<double>(nrows, nitems, (const int4*)items, rowptr, ci, val, X, ldx, k, beta, Y, ldy, lg,
                               (cudaStream_t)stream);
}
SP3_API int sp3_cuda_rows_f32(int mode, long long n, const long long* idx, const float* src, long long lds,
                              float* dst, long long ldd, int k, void* stream) {
    return launch_rows<float>(mode, n, idx, src, lds, dst, ldd, k, (cudaStream_t)stream);
}
SP3_API int sp3_cuda_rows_f64(int mode, long long n, const long long* idx, const double* src, long long lds,
                              double* dst, long long ldd, int k, void* stream) {
    return launch_rows<double>(mode, n, idx, src, lds, dst, ldd, k, (cudaStream_t)stream);
}
SP3_API int sp3_cuda_fill_rows_f32(const long long* gid, long long nrows, long long col0, int ncols, long long ld,
                                   long long kglobal, int kind, double cval, unsigned long long seed,
                                   unsigned long long stream_id, float* out, void* stream) {
    const long long n = nrows * ncols;
    if (n == 0) return 0;
    fill_rows_kernel<float><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gid, nrows, col0, ncols, ld, kglobal, kind, cval, seed, stream_id, out);
    return (int)cudaGetLastError();
}
SP3_API int sp3_cuda_fill_rows_f64(const long long* gid, long long nrows, long long col0, int ncols, long long ld,
                                   long long kglobal, int kind, double cval, unsigned long long seed,
                                   unsigned long long stream_id, double* out, void* stream) {
    const long long n = nrows * ncols;
    if (n == 0) return 0;
    fill_rows_kernel<double><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gid, nrows, col0, ncols, ld, kglobal, kind, cval, seed, stream_id, out);
    return (int)cudaGetLastError();
}
// part must hold 1024 doubles of scratch; out one double.
SP3_API int sp3_cuda_sum_f32(const float* x, long long n, double* part, double* out, void* stream) {
    sum_stage1<float><<<1024, 256, 0, (cudaStream_t)stream>>>(x, n, part);
    sum_stage2<<<1, 256, 0, (cudaStream_t)stream>>>(part, 1024, out);
    return (int)cudaGetLastError();
}
SP3_API int sp3_cuda_sum_f64(const double* x, long long n, double* part, double* out, void* stream) {
    sum_stage1<double><<<1024, 256, 0, (cudaStream_t)stream>>>(x, n, part);
    sum_stage2<<<1, 256, 0, (cudaStream_t)stream>>>(part, 1024, out);
    return (int)cudaGetLastError();
}
SP3_API int sp3_cuda_check_range(long long n, const int* idx, int limit, int which, int* status, void* stream) {
    if (n == 0) return 0;
    check_range_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, idx, limit, which, status);
    return (int)cudaGetLastError();
}
SP3_API int sp3_cuda_remap(long long n, const int* idx, const int* table, long long table_len, int* out,
                           int* status, void* stream) {
    if (n == 0) return 0;
    remap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, idx, table, table_len, out, status);
    return (int)cudaGetLastError();
}
SP3_API int sp3_cuda_invert_perm(long long n, const long long* perm, long long* inv, int* status, void* stream) {
    if (n == 0) return 0;
    invert_perm_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, perm, inv, status);
    return (int)cudaGetLastError();
}
SP3_API int sp3_cuda_touch_masks(long long nnz, const int* rows, const int* cols, const int* rowmap,
                                 const int* colmap, void* row_mask, void* col_mask, void* stream) {
    if (nnz == 0) return 0;
    touch_masks_kernel<<<(unsigned)((nnz + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        nnz, rows, cols, rowmap, colmap, (unsigned long long*)row_mask, (unsigned long long*)col_mask);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// SpMM entry point that allocates nothing (declared in sp3_noalloc.h).
//
// The scheduled SpMM kernel needs scratch for rows that are split into
// pieces: one partial row per piece plus one arrival counter per split row.
// Callers that are not allowed to call cudaMalloc (see the header) get that
// scratch from the fixed array below instead of from an allocation.  The
// array is part of the loaded library image: every GPU that loads the library
// holds SP3_NOALLOC_SCRATCH_BYTES of device memory until the process exits.
// ---------------------------------------------------------------------------
#include <atomic>

#include "sp3_noalloc.h"

namespace {
static __device__ __align__(256) unsigned char g_noalloc_scratch[SP3_NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
// Device address of g_noalloc_scratch per device ordinal, filled on the first
// call made with that device current.  In host code the symbol name itself is
// only a handle; the address has to come from cudaGetSymbolAddress.  Atomic
// because first calls may come from several host threads at once (they would
// all store the same address).
std::atomic<unsigned char*> g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
}  // namespace

SP3_API int sp3_cuda_spmm_f32_noalloc(int nrows, int nitems, const void* items, const long long* rowptr,
                                      const int* colidx, const float* val, const float* X, long long ldx, int k,
                                      float beta, float* Y, long long ldy, const int* first_piece,
                                      const int* npieces, int nlong, int total_pieces, int piece_len,
                                      void* stream) {
    if (nrows < 0 || nitems < 0 || nlong < 0 || total_pieces < 0 || k <= 0) return SP3_NOALLOC_E_ARG;
    // layout of the scratch: [counters: SP3_NOALLOC_MAX_SPLIT_ROWS x int32][carry: total_pieces x ldc floats]
    const long long ldc = ((long long)k + 3) / 4 * 4;  // keep carry rows 16-byte aligned
    const size_t counters_bytes = (size_t)SP3_NOALLOC_MAX_SPLIT_ROWS * sizeof(int);
    const size_t carry_bytes = (size_t)total_pieces * (size_t)ldc * sizeof(float);
    if (nlong > SP3_NOALLOC_MAX_SPLIT_ROWS || counters_bytes + carry_bytes > (size_t)SP3_NOALLOC_SCRATCH_BYTES)
        return SP3_NOALLOC_E_TOO_LARGE;
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return (int)err;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return SP3_NOALLOC_E_ARG;
    unsigned char* base = g_noalloc_ptr[dev].load(std::memory_order_relaxed);
    if (!base) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (err != cudaSuccess) return (int)err;
        base = (unsigned char*)p;
        g_noalloc_ptr[dev].store(base, std::memory_order_relaxed);
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (nlong > 0) {
        // the array keeps whatever the previous call left; counters must start at zero
        err = cudaMemsetAsync(base, 0, (size_t)nlong * sizeof(int), st);
        if (err != cudaSuccess) return (int)err;
    }
    sp3::SpmmLong lg{first_piece, npieces, (int*)base, (void*)(base + counters_bytes), ldc, piece_len, nullptr};
    return sp3::launch_spmm<float>(nrows, nitems, (const int4*)items, rowptr, colidx, val, X, ldx, k, beta, Y, ldy,
                                   lg, st);
}

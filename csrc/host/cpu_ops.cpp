// CPU local kernels (fp32 and fp64): SDDMM, SpMM, row gather / scatter /
// scatter-add and checksum.  They serve the CPU (gloo) pipeline and act as the
// plain reference loops the CUDA kernels are tested against.
//
// Same math as the reference loops src/core_ops.cpp:5-35 and the staging copies
// src/comm.hpp:90-103,166-189, without per-element bounds checks, over a
// row-sorted nonzero list, threaded with OpenMP.
#include "sp3_host.hpp"

#include <cstring>

namespace {
template <typename T>
int sddmm_impl(int64_t nnz, const int32_t* rowidx, const int32_t* colidx, const T* sval,
               const T* A, int64_t lda, const T* B, int64_t ldb, int64_t k, T* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nnz; ++i) {
        const T* a = A + (int64_t)rowidx[i] * lda;
        const T* b = B + (int64_t)colidx[i] * ldb;
        T acc = 0;
        for (int64_t j = 0; j < k; ++j) acc += a[j] * b[j];
        out[i] = sval ? acc * sval[i] : acc;
    }
    return sp3::OK;
}

template <typename T>
int spmm_impl(int64_t nrows, const int64_t* rowptr, const int32_t* colidx, const T* val,
              const T* X, int64_t ldx, int64_t k, T beta, T* Y, int64_t ldy) {
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t r = 0; r < nrows; ++r) {
        T* y = Y + r * ldy;
        if (beta == (T)0) std::memset(y, 0, (size_t)k * sizeof(T));
        else if (beta != (T)1) for (int64_t j = 0; j < k; ++j) y[j] *= beta;
        for (int64_t p = rowptr[r]; p < rowptr[r + 1]; ++p) {
            const T* x = X + (int64_t)colidx[p] * ldx;
            const T v = val[p];
            for (int64_t j = 0; j < k; ++j) y[j] += v * x[j];
        }
    }
    return sp3::OK;
}

// mode 0: dst[i] = src[idx[i]] (gather / pack); 1: dst[idx[i]] = src[i]
// (scatter / unpack); 2: dst[idx[i]] += src[i] (scatter-add; idx must not
// repeat inside one call, which holds for per-peer row lists).
template <typename T>
int rows_impl(int mode, int64_t n, const int64_t* idx, const T* src, int64_t lds, T* dst,
              int64_t ldd, int64_t k) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        if (mode == 0) std::memcpy(dst + i * ldd, src + idx[i] * lds, (size_t)k * sizeof(T));
        else if (mode == 1) std::memcpy(dst + idx[i] * ldd, src + i * lds, (size_t)k * sizeof(T));
        else { T* d = dst + idx[i] * ldd; const T* s = src + i * lds; for (int64_t j = 0; j < k; ++j) d[j] += s[j]; }
    }
    return sp3::OK;
}
}  // namespace

SP3_API int sp3_cpu_sddmm_f32(int64_t nnz, const int32_t* ri, const int32_t* ci, const float* sv,
                              const float* A, int64_t lda, const float* B, int64_t ldb, int64_t k, float* out) {
    return sddmm_impl<float>(nnz, ri, ci, sv, A, lda, B, ldb, k, out);
}
SP3_API int sp3_cpu_sddmm_f64(int64_t nnz, const int32_t* ri, const int32_t* ci, const double* sv,
                              const double* A, int64_t lda, const double* B, int64_t ldb, int64_t k, double* out) {
    return sddmm_impl<double>(nnz, ri, ci, sv, A, lda, B, ldb, k, out);
}
SP3_API int sp3_cpu_spmm_f32(int64_t nrows, const int64_t* rowptr, const int32_t* ci, const float* v,
                             const float* X, int64_t ldx, int64_t k, float beta, float* Y, int64_t ldy) {
    return spmm_impl<float>(nrows, rowptr, ci, v, X, ldx, k, beta, Y, ldy);
}
SP3_API int sp3_cpu_spmm_f64(int64_t nrows, const int64_t* rowptr, const int32_t* ci, const double* v,
                             const double* X, int64_t ldx, int64_t k, double beta, double* Y, int64_t ldy) {
    return spmm_impl<double>(nrows, rowptr, ci, v, X, ldx, k, beta, Y, ldy);
}
SP3_API int sp3_cpu_rows_f32(int mode, int64_t n, const int64_t* idx, const float* src, int64_t lds,
                             float* dst, int64_t ldd, int64_t k) {
    return rows_impl<float>(mode, n, idx, src, lds, dst, ldd, k);
}
SP3_API int sp3_cpu_rows_f64(int mode, int64_t n, const int64_t* idx, const double* src, int64_t lds,
                             double* dst, int64_t ldd, int64_t k) {
    return rows_impl<double>(mode, n, idx, src, lds, dst, ldd, k);
}

// Seeded synthetic matrix and operand generators.
//
// The reference only has an unseeded unique-(r,c) generator with value 1.0
// (src/SparseMatrix.hpp:49-67) and fills dense operands with a constant
// (miniapp/bench_both.cpp:189-192).  Here every value is a pure function of
// (seed, stream, index), so all ranks can build the same global matrix, or
// just their own part of it, without communicating.
#include "sp3_host.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <parallel/algorithm>
#endif

namespace sp3 {
double normal01(uint64_t seed, uint64_t stream, uint64_t idx) {
    double u1 = u01(rnd(seed, stream, 2 * idx));
    double u2 = u01(rnd(seed, stream, 2 * idx + 1));
    if (u1 < 1e-300) u1 = 1e-300;
    return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
}
}  // namespace sp3

namespace {
enum Stream : uint64_t { S_COL = 11, S_VAL = 12, S_DEG = 13, S_RMAT = 14, S_REDRAW = 15 };

// Fills cols[0..d) with d distinct values in [0,N), ascending.
void draw_distinct(uint64_t seed, uint64_t row, uint32_t d, uint64_t N, uint32_t* cols) {
    if ((uint64_t)d * 2 > N) {
        // dense row: partial Fisher-Yates over the whole column range
        std::vector<uint32_t> all(N);
        for (uint64_t i = 0; i < N; ++i) all[i] = (uint32_t)i;
        for (uint32_t s = 0; s < d; ++s) {
            uint64_t j = s + sp3::rnd(seed, S_COL, row * 0x100000001B3ull + s) % (N - s);
            std::swap(all[s], all[j]);
            cols[s] = all[s];
        }
        std::sort(cols, cols + d);
        return;
    }
    for (uint32_t s = 0; s < d; ++s)
        cols[s] = (uint32_t)(sp3::rnd(seed, S_COL, row * 0x100000001B3ull + s) % N);
    for (uint64_t attempt = 1;; ++attempt) {
        std::sort(cols, cols + d);
        bool dup = false;
        for (uint32_t s = 1; s < d; ++s)
            if (cols[s] == cols[s - 1]) {
                dup = true;
                cols[s - 1] = (uint32_t)(sp3::rnd(seed ^ attempt, S_REDRAW, row * 0x100000001B3ull + s) % N);
            }
        if (!dup) return;
    }
}
}  // namespace

// Every row gets exactly `deg` distinct uniform columns (ascending); values U(0,1).
SP3_API int sp3_gen_fixed_degree(uint64_t M, uint64_t N, uint32_t deg, uint64_t seed,
                                 uint32_t* rows, uint32_t* cols, double* vals) {
    if (deg > N) return sp3::E_ARG;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)M; ++r) {
        uint32_t* c = cols + (uint64_t)r * deg;
        draw_distinct(seed, (uint64_t)r, deg, N, c);
        for (uint32_t s = 0; s < deg; ++s) {
            rows[(uint64_t)r * deg + s] = (uint32_t)r;
            vals[(uint64_t)r * deg + s] = sp3::u01(sp3::rnd(seed, S_VAL, (uint64_t)r * deg + s));
        }
    }
    return sp3::OK;
}

// Row degrees.  kind 0: Zipf-like power law, d = floor(u^(-1/(alpha-1)))
// clipped to [dmin,dmax] (P(d >= x) = x^-(alpha-1)); kind 1: Poisson(mean),
// the row-degree law of an Erdos-Renyi matrix with N*p = mean, clipped to
// [0, dmax].
SP3_API int sp3_gen_degrees(uint64_t M, int kind, double param, uint32_t dmin, uint32_t dmax,
                            uint64_t seed, uint32_t* deg) {
    if (kind == 0 && param <= 1.0) return sp3::E_ARG;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)M; ++r) {
        double u = sp3::u01(sp3::rnd(seed, S_DEG, (uint64_t)r));
        double d;
        if (kind == 0) {
            if (u < 1e-18) u = 1e-18;
            d = std::floor(std::pow(u, -1.0 / (param - 1.0)));
        } else {
            // inverse-CDF Poisson; fine for the means used here (< ~700)
            double p = std::exp(-param), cdf = p;
            uint32_t k = 0;
            while (u > cdf && k < dmax) { ++k; p *= param / k; cdf += p; }
            d = k;
        }
        if (d < dmin) d = dmin;
        if (d > dmax) d = dmax;
        deg[r] = (uint32_t)d;
    }
    return sp3::OK;
}

// Given rowptr (prefix sum of degrees), fills rows/cols/vals: deg[r] distinct
// uniform columns per row, ascending; values U(0,1).
SP3_API int sp3_gen_from_rowptr(uint64_t M, uint64_t N, const uint64_t* rowptr, uint64_t seed,
                                uint32_t* rows, uint32_t* cols, double* vals) {
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 4096)
    for (int64_t r = 0; r < (int64_t)M; ++r) {
        uint64_t b = rowptr[r], e = rowptr[r + 1];
        if (e - b > N) { bad = 1; continue; }
        draw_distinct(seed, (uint64_t)r, (uint32_t)(e - b), N, cols + b);
        for (uint64_t i = b; i < e; ++i) {
            rows[i] = (uint32_t)r;
            vals[i] = sp3::u01(sp3::rnd(seed, S_VAL, i));
        }
    }
    return bad ? sp3::E_ARG : sp3::OK;
}

// The same matrix as sp3_gen_from_rowptr restricted to one block of a 2D partition: rows with rowmap[r] == x,
// columns with colmap[c] == y (a null map keeps everything on that side).  Every entry has the value it has in
// the whole matrix (values are drawn by global position), so ranks that each generate their own block hold,
// together, exactly the matrix a single generator call would give.  Two calls: with rows == null only the number
// of entries is returned in *count; then the arrays of that length are filled (row-major, columns ascending).
SP3_API int sp3_gen_from_rowptr_block(uint64_t M, uint64_t N, const uint64_t* rowptr, uint64_t seed,
                                      const int32_t* rowmap, int32_t x, const int32_t* colmap, int32_t y,
                                      uint64_t* count, uint32_t* rows, uint32_t* cols, double* vals) {
    std::vector<uint64_t> start(M + 1, 0);
    int bad = 0;
#pragma omp parallel
    {
        std::vector<uint32_t> tmp;
#pragma omp for schedule(dynamic, 4096)
        for (int64_t r = 0; r < (int64_t)M; ++r) {
            if (rowmap && rowmap[r] != x) continue;
            const uint64_t b = rowptr[r], e = rowptr[r + 1];
            if (e - b > N) { bad = 1; continue; }
            if (!colmap) { start[r + 1] = e - b; continue; }
            tmp.resize(e - b);
            draw_distinct(seed, (uint64_t)r, (uint32_t)(e - b), N, tmp.data());
            uint64_t kept = 0;
            for (uint64_t s = 0; s < e - b; ++s) kept += colmap[tmp[s]] == y;
            start[r + 1] = kept;
        }
    }
    if (bad) return sp3::E_ARG;
    for (uint64_t r = 0; r < M; ++r) start[r + 1] += start[r];
    *count = start[M];
    if (!rows) return sp3::OK;
#pragma omp parallel
    {
        std::vector<uint32_t> tmp;
#pragma omp for schedule(dynamic, 4096)
        for (int64_t r = 0; r < (int64_t)M; ++r) {
            if (start[r + 1] == start[r]) continue;
            const uint64_t b = rowptr[r], e = rowptr[r + 1];
            tmp.resize(e - b);
            draw_distinct(seed, (uint64_t)r, (uint32_t)(e - b), N, tmp.data());
            uint64_t o = start[r];
            for (uint64_t s = 0; s < e - b; ++s) {
                if (colmap && colmap[tmp[s]] != y) continue;
                rows[o] = (uint32_t)r;
                cols[o] = tmp[s];
                vals[o] = sp3::u01(sp3::rnd(seed, S_VAL, b + s));
                ++o;
            }
        }
    }
    return sp3::OK;
}

// R-MAT edge keys (row << 32 | col) for a 2^scale square graph; `nedges`
// edges are drawn by `scale` quadrant choices with probabilities a,b,c,(d).
// The caller removes duplicates with sp3_sort_unique_u64.
SP3_API int sp3_gen_rmat_keys(uint32_t scale, uint64_t nedges, double a, double b, double c,
                              uint64_t seed, uint64_t* keys) {
    if (scale == 0 || scale > 31) return sp3::E_ARG;
    const double ab = a + b, abc = a + b + c;
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < (int64_t)nedges; ++e) {
        uint64_t r = 0, col = 0;
        for (uint32_t l = 0; l < scale; ++l) {
            double u = sp3::u01(sp3::rnd(seed, S_RMAT + l, (uint64_t)e));
            uint64_t rb = (u >= ab), cb = (u >= a && u < ab) || (u >= abc);
            r = (r << 1) | rb;
            col = (col << 1) | cb;
        }
        keys[e] = (r << 32) | col;
    }
    return sp3::OK;
}

SP3_API int64_t sp3_sort_unique_u64(uint64_t* keys, uint64_t n) {
#ifdef _OPENMP
    __gnu_parallel::sort(keys, keys + n);
#else
    std::sort(keys, keys + n);
#endif
    return (int64_t)(std::unique(keys, keys + n) - keys);
}

// Splits sorted keys into rows/cols and draws U(0,1) values by position.
SP3_API int sp3_keys_to_coo(const uint64_t* keys, uint64_t n, uint64_t seed,
                            uint32_t* rows, uint32_t* cols, double* vals) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        rows[i] = (uint32_t)(keys[i] >> 32);
        cols[i] = (uint32_t)(keys[i] & 0xFFFFFFFFull);
        vals[i] = sp3::u01(sp3::rnd(seed, S_VAL, (uint64_t)i));
    }
    return sp3::OK;
}

// Dense operand rows: out[i, j] = f(seed, stream, gid[i], col0 + j) for
// j < ncols, with leading dimension ld.  kind 0: N(0,1); kind 1: gid/1000
// (the fill of the reference's checkers, miniapp/numCheckSeq.cpp:125-128);
// kind 2: constant `cval`.  The CUDA twin of this function uses the same
// counter scheme so host- and device-filled operands agree to rounding.
SP3_API int sp3_fill_rows_f64(const int64_t* gid, uint64_t nrows, uint64_t col0, uint64_t ncols,
                              uint64_t ld, uint64_t kglobal, int kind, double cval, uint64_t seed,
                              uint64_t stream, double* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)nrows; ++i)
        for (uint64_t j = 0; j < ncols; ++j) {
            double v;
            if (kind == 0) v = sp3::normal01(seed, stream, (uint64_t)gid[i] * kglobal + col0 + j);
            else if (kind == 1) v = (double)gid[i] / 1000.0;
            else v = cval;
            out[(uint64_t)i * ld + j] = v;
        }
    return sp3::OK;
}

SP3_API int sp3_fill_rows_f32(const int64_t* gid, uint64_t nrows, uint64_t col0, uint64_t ncols,
                              uint64_t ld, uint64_t kglobal, int kind, double cval, uint64_t seed,
                              uint64_t stream, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)nrows; ++i)
        for (uint64_t j = 0; j < ncols; ++j) {
            double v;
            if (kind == 0) v = sp3::normal01(seed, stream, (uint64_t)gid[i] * kglobal + col0 + j);
            else if (kind == 1) v = (double)gid[i] / 1000.0;
            else v = cval;
            out[(uint64_t)i * ld + j] = (float)v;
        }
    return sp3::OK;
}

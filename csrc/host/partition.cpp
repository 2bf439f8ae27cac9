// 2D nonzero partition, touch masks, dense-row ownership and CSR ordering.
//
// What the reference does with a rank-0 shuffle + Bcast (src/parallel_io.hpp:
// 64-79), per-nonzero bucketing (:95-105), a directory exchange of touched ids
// (src/distribute.cpp:27-163) and hash-map index compaction
// (src/SparseMatrix.hpp:69-99) is restated here around one idea: a 64-bit
// *touch mask* per global row (bit y set when mesh-column y holds a nonzero of
// that row) and per global column (bit x).  Masks from different ranks combine
// with a plain sum/or, and owners, per-peer need lists and send lists are all
// pure functions of (map, mask, seed) that every rank evaluates locally.
#include "sp3_host.hpp"

#include <algorithm>
#include <cstring>
#include <numeric>
#include <omp.h>
#include <vector>

// map[id] = mesh coordinate in [0,parts): seeded Fisher-Yates shuffle of the
// ids followed by round-robin assignment (parallel_io.hpp:64-76).
SP3_API int sp3_rr_map(uint64_t n, uint32_t parts, uint64_t seed, uint64_t stream, int32_t* map) {
    if (parts == 0) return sp3::E_ARG;
    std::vector<uint32_t> perm(n);
    std::iota(perm.begin(), perm.end(), 0u);
    for (uint64_t i = n; i > 1; --i) {
        uint64_t j = sp3::rnd(seed, stream, i) % i;
        std::swap(perm[i - 1], perm[j]);
    }
    for (uint64_t i = 0; i < n; ++i) map[perm[i]] = (int32_t)(i % parts);
    return sp3::OK;
}

// Stable bucketing of nonzeros by destination block b = rowmap[r]*Y + colmap[c].
// offsets has X*Y+1 entries; perm lists source positions block by block, in
// source order inside a block.
SP3_API int sp3_bucket_blocks(uint64_t nnz, const uint32_t* rows, const uint32_t* cols,
                              const int32_t* rowmap, const int32_t* colmap, uint32_t X, uint32_t Y,
                              int64_t* offsets, int64_t* perm) {
    const uint32_t nb = X * Y;
    // Every thread counts a contiguous piece of the nonzeros; the piece counts, scanned block-major and
    // thread-minor, give each thread its write positions, so the result is the stable order whatever the
    // number of threads.
    const int T = std::max(1, omp_get_max_threads());
    std::vector<int64_t> cnt((size_t)T * nb, 0);
    int bad = 0;
#pragma omp parallel num_threads(T) reduction(| : bad)
    {
        const int t = omp_get_thread_num();
        const uint64_t lo = nnz * (uint64_t)t / T, hi = nnz * (uint64_t)(t + 1) / T;
        int64_t* c = cnt.data() + (size_t)t * nb;
        for (uint64_t i = lo; i < hi; ++i) {
            uint32_t b = (uint32_t)rowmap[rows[i]] * Y + (uint32_t)colmap[cols[i]];
            if (b >= nb) { bad = 1; break; }
            ++c[b];
        }
    }
    if (bad) return sp3::E_RANGE;
    int64_t run = 0;
    for (uint32_t b = 0; b < nb; ++b) {
        offsets[b] = run;
        for (int t = 0; t < T; ++t) { int64_t c = cnt[(size_t)t * nb + b]; cnt[(size_t)t * nb + b] = run; run += c; }
    }
    offsets[nb] = run;
    if (!perm) return sp3::OK;
#pragma omp parallel num_threads(T)
    {
        const int t = omp_get_thread_num();
        const uint64_t lo = nnz * (uint64_t)t / T, hi = nnz * (uint64_t)(t + 1) / T;
        int64_t* c = cnt.data() + (size_t)t * nb;
        for (uint64_t i = lo; i < hi; ++i) {
            uint32_t b = (uint32_t)rowmap[rows[i]] * Y + (uint32_t)colmap[cols[i]];
            perm[c[b]++] = (int64_t)i;
        }
    }
    return sp3::OK;
}

// row_mask[r] |= 1 << colmap[c], col_mask[c] |= 1 << rowmap[r] for every
// nonzero given.  Works on the whole matrix or on one rank's block (then only
// that rank's own bit appears and masks are summed across the mesh).
SP3_API int sp3_touch_masks(uint64_t nnz, const uint32_t* rows, const uint32_t* cols,
                            const int32_t* rowmap, const int32_t* colmap,
                            int64_t* row_mask, int64_t* col_mask) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)nnz; ++i) {
        uint32_t r = rows[i], c = cols[i];
        int64_t rb = (int64_t)1 << colmap[c], cb = (int64_t)1 << rowmap[r];
        if (!(__atomic_load_n(&row_mask[r], __ATOMIC_RELAXED) & rb))
            __atomic_fetch_or(&row_mask[r], rb, __ATOMIC_RELAXED);
        if (!(__atomic_load_n(&col_mask[c], __ATOMIC_RELAXED) & cb))
            __atomic_fetch_or(&col_mask[c], cb, __ATOMIC_RELAXED);
    }
    return sp3::OK;
}

// Owner choice ("respect communication", distribute.cpp:107-150): the owner
// coordinate of id i along the free mesh axis is a seeded pick among the set
// bits of mask[i]; ids nobody touches are dealt round-robin inside their mesh
// line (distribute.cpp:135-146).  policy 1 ignores the masks and deals all
// ids round-robin (the reference's unused random scheme, distribute.cpp:
// 212-247).  Also returns pos[i], the index of id i inside its owner's
// ascending owned list, and counts[line*parts + owner] = owned list lengths.
SP3_API int sp3_assign_owners(uint64_t n, const int64_t* mask, const int32_t* linemap,
                              uint32_t nlines, uint32_t parts, int policy, uint64_t seed,
                              uint64_t stream, int32_t* owner, int32_t* pos, int64_t* counts) {
    if (parts == 0 || parts > 62) return sp3::E_ARG;
    // pass 1 (parallel): the seeded pick among the touching ranks depends on the id alone
    int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        if ((uint32_t)linemap[i] >= nlines) { bad = 1; owner[i] = -1; continue; }
        uint64_t m = policy == 1 ? 0 : (uint64_t)mask[i];
        if (m == 0) { owner[i] = -1; continue; }
        int pc = __builtin_popcountll(m);
        int pick = (int)(sp3::rnd(seed, stream, (uint64_t)i) % (uint64_t)pc);
        uint64_t mm = m;
        while (pick--) mm &= mm - 1;
        int o = __builtin_ctzll(mm);
        if ((uint32_t)o >= parts) { bad = 1; o = -1; }
        owner[i] = o;
    }
    if (bad) return sp3::E_RANGE;
    // pass 2 (in id order): round-robin for the ids nobody touches, positions inside the owned lists
    std::vector<uint64_t> rr(nlines, 0);
    std::fill(counts, counts + (size_t)nlines * parts, 0);
    for (uint64_t i = 0; i < n; ++i) {
        uint32_t line = (uint32_t)linemap[i];
        if (owner[i] < 0) owner[i] = (int32_t)(rr[line]++ % parts);
        pos[i] = (int32_t)counts[(size_t)line * parts + owner[i]]++;
    }
    return sp3::OK;
}

// Orders local nonzeros by (local row, local col) and builds the CSR row
// pointer.  perm[i] is the source position of the i-th nonzero in CSR order.
SP3_API int sp3_csr_order(uint64_t nnz, const int32_t* lrow, const int32_t* lcol, uint64_t nrows,
                          int64_t* rowptr, int64_t* perm) {
    std::vector<int64_t> cnt(nrows + 1, 0);
    for (uint64_t i = 0; i < nnz; ++i) {
        if (lrow[i] < 0 || (uint64_t)lrow[i] >= nrows) return sp3::E_RANGE;
        ++cnt[lrow[i] + 1];
    }
    for (uint64_t r = 0; r < nrows; ++r) cnt[r + 1] += cnt[r];
    std::memcpy(rowptr, cnt.data(), (nrows + 1) * sizeof(int64_t));
    for (uint64_t i = 0; i < nnz; ++i) perm[cnt[lrow[i]]++] = (int64_t)i;
#pragma omp parallel for schedule(dynamic, 1024)
    for (int64_t r = 0; r < (int64_t)nrows; ++r) {
        int64_t b = rowptr[r], e = rowptr[r + 1];
        if (e - b > 1)
            std::sort(perm + b, perm + e, [&](int64_t a, int64_t c) {
                return lcol[a] != lcol[c] ? lcol[a] < lcol[c] : a < c;
            });
    }
    return sp3::OK;
}

// out[i] = table[idx[i]] with a range check: the index rewrite of
// ReMapIndices / localizeIndices (SparseMatrix.hpp:69-106) as one pass.
SP3_API int sp3_remap_u32(uint64_t n, const uint32_t* idx, const int32_t* table, uint64_t table_len,
                          int32_t* out) {
    int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        if (idx[i] >= table_len || table[idx[i]] < 0) { bad = 1; out[i] = -1; }
        else out[i] = table[idx[i]];
    }
    return bad ? sp3::E_RANGE : sp3::OK;
}

// Counts rows and columns without any nonzero (tools/countEmptyRows.cpp:80-92).
SP3_API int sp3_count_empty(uint64_t nnz, const uint32_t* rows, const uint32_t* cols,
                            uint64_t nrows, uint64_t ncols, uint64_t* empty_rows, uint64_t* empty_cols) {
    std::vector<uint8_t> rs(nrows, 0), cs(ncols, 0);
    for (uint64_t i = 0; i < nnz; ++i) {
        if (rows[i] >= nrows || cols[i] >= ncols) return sp3::E_RANGE;
        rs[rows[i]] = 1; cs[cols[i]] = 1;
    }
    uint64_t er = 0, ec = 0;
    for (auto v : rs) er += !v;
    for (auto v : cs) ec += !v;
    *empty_rows = er; *empty_cols = ec;
    return sp3::OK;
}

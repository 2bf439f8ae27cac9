// Warp-level bodies of the SDDMM and SpMM kernels, shared by the local
// kernels (local_ops.cu) and the fused compute+communication kernels
// (fused_impl.cuh).  Where dense rows come from and where results go is a
// template policy, so both families run the same inner loops:
//
//   SDDMM   A rows:  RowsByStride (one local block) | RowsByPeerRef (rows that
//                    stay in their owners' memory, local or peer)
//           output:  StoreLocal | the fused kernel's slice-routing store
//   SpMM    emit:    EmitLocal (Y = beta*Y + acc) | the fused kernel's
//                    owned-or-push emit
//
// Reference loops: src/core_ops.cpp:5-35.
#pragma once
#include "sp3_cuda.cuh"

namespace sp3 {

constexpr int SDDMM_PER_SLOT = 32;  // nonzeros per lane group; multiple of every G

// Tuning knobs (compile time): resident 256-thread blocks per SM the SDDMM
// kernels are compiled for, and whether the loop over the sub-batches of an
// index batch is unrolled (more loads in flight per warp, more registers).
#ifndef SP3_SDDMM_MINB
#define SP3_SDDMM_MINB 4
#endif
// With more than two vectors per lane the row registers alone need the larger budget of two blocks per SM.
constexpr int sddmm_min_blocks(int R) { return R <= 2 ? SP3_SDDMM_MINB : 2; }
#ifndef SP3_SDDMM_UNROLL_BATCH
#define SP3_SDDMM_UNROLL_BATCH 1
#endif

template <int G> __device__ __forceinline__ unsigned group_mask(int slot) {
    return G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (slot * G));
}

// Sums N values per lane across a group of G lanes with a halving butterfly:
// at each step a lane keeps one half of its values and hands the other half
// to its partner, so the whole reduction costs N-1 + log2(G/N) shuffles instead
// of N*log2(G).  N <= G, both powers of two.  On return v[0] of lane gl holds
// the group total of value number gl / (G/N).
template <typename T, int G, int N>
__device__ __forceinline__ void group_transpose_reduce(T (&v)[N], unsigned gmask, int gl) {
    int n = N;
#pragma unroll
    for (int m = G / 2; m > 0; m >>= 1) {
        if (n > 1) {
            const int half = n >> 1;
            const bool upper = (gl & m) != 0;
#pragma unroll
            for (int t = 0; t < N / 2; ++t) {
                if (t < half) {
                    const T send = upper ? v[t] : v[t + half];
                    const T keep = upper ? v[t + half] : v[t];
                    v[t] = keep + __shfl_xor_sync(gmask, send, m, G);
                }
            }
            n = half;
        } else {
            v[0] += __shfl_xor_sync(gmask, v[0], m, G);
        }
    }
}

// ---- dense-row loads ----------------------------------------------------------
// NC = true: the non-coherent read-only path (ld.global.nc), for operands that no thread writes while the
// kernel runs (the local kernels).  NC = false: an ordinary load.  The fused kernels use it for every dense
// row, because rows of the pulled part of a block are written by other warps of the same launch; ordinary
// loads are ordered after the acquire that tells a warp the rows are there, the read-only path is not.
template <bool NC, typename V> __device__ __forceinline__ V ld_row(const V* p) {
    if constexpr (NC) return __ldg(p);
    else return *p;
}

// ---- row access policies ---------------------------------------------------
// A policy turns the local row index of a nonzero into a 31-bit *reference*
// (`ref`, evaluated by every lane for its own nonzero when a batch of indices
// is read, so a table lookup is off the critical path) and a reference into
// the address of the dense row (`resolve`, pure arithmetic).  The reference is
// what the lane group passes round by shuffle and compares to detect a row
// change.
template <typename T> struct RowsByStride {
    using V = typename Vec<T>::type;
    const V* base;
    long long ld_v;
    __device__ __forceinline__ int ref(int row) const { return row; }
    __device__ __forceinline__ const V* resolve(int r) const { return base + (long long)r * ld_v; }
};
// Rows that live in the owners' heaps: reference = owner rank (6 bits) and row
// number inside the owner's block (25 bits); `bases` (shared memory) holds the
// block address of every rank as mapped into this process.
constexpr int PEER_REF_SHIFT = 25;
template <typename T> struct RowsByPeerRef {
    using V = typename Vec<T>::type;
    const int* table;                  // [local rows] references; null: every row is in this rank's own block
    const unsigned long long* bases;   // [ranks] block base addresses
    unsigned long long row_bytes;
    int self_bits;                     // this rank << PEER_REF_SHIFT (used when table is null)
    __device__ __forceinline__ int ref(int row) const { return table ? __ldg(table + row) : (self_bits | row); }
    __device__ __forceinline__ const V* resolve(int r) const {
        return reinterpret_cast<const V*>(bases[r >> PEER_REF_SHIFT] +
                                          (unsigned long long)(r & ((1 << PEER_REF_SHIFT) - 1)) * row_bytes);
    }
};

template <typename T> struct StoreLocal {
    T* out;
    const T* sval;
    const int* orig;  // optional: result position of nonzero i (null: i)
    __device__ __forceinline__ void operator()(long long i, T dot) const {
        const T v = sval ? dot * __ldg(sval + i) : dot;
        if (orig) out[__ldg(orig + i)] = v;
        else out[i] = v;
    }
};

// ---------------------------------------------------------------------------
// SDDMM work unit of one warp: 32/G lane groups x SDDMM_PER_SLOT consecutive
// nonzeros each, starting at nonzero `unit * (32/G) * SDDMM_PER_SLOT`.
// A group reads its (row, col) pairs G at a time with one coalesced load per
// array and hands them round with in-group shuffles; each lane holds R
// 16-byte vectors of a dense row, so a dot product costs R vector loads and 4R
// FMAs per lane, and U dot products are reduced together with the butterfly
// above.  The list is sorted by row, so the A row stays in registers until
// the row changes.  Results leave as one coalesced store per G nonzeros.
// ---------------------------------------------------------------------------
template <typename T, int G, int R, int U, typename ARows, typename Store, bool NC = true>
__device__ __forceinline__ void sddmm_warp_unit(long long unit, long long nnz, const int* __restrict__ rowidx,
                                                const int* __restrict__ colidx, const ARows& arows,
                                                const typename Vec<T>::type* __restrict__ Bv, long long ldb_v,
                                                int nvec, const Store& store, int lane) {
    using V = typename Vec<T>::type;
    constexpr int SLOTS = 32 / G;
    constexpr int UU = U < G ? U : G;
    const int slot = lane / G, gl = lane % G;
    const unsigned gmask = group_mask<G>(slot);
    const long long begin = (unit * SLOTS + slot) * (long long)SDDMM_PER_SLOT;
    int cur_row = -1;
    V a[R];
#pragma unroll
    for (int r = 0; r < R; ++r) a[r] = vzero((V*)nullptr);
    for (int base = 0; base < SDDMM_PER_SLOT; base += G) {
        const long long i = begin + base + gl;
        const bool ok = i < nnz;
        const int my_r = ok ? arows.ref(__ldg(rowidx + i)) : -1;
        const int my_c = ok ? __ldg(colidx + i) : -1;
        T my_out = 0;
#if SP3_SDDMM_UNROLL_BATCH
#pragma unroll
#else
#pragma unroll 1
#endif
        for (int j = 0; j < G; j += UU) {
            int rr[UU], cc[UU];
            V b[UU][R];
            T acc[UU];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                rr[u] = __shfl_sync(gmask, my_r, j + u, G);
                cc[u] = __shfl_sync(gmask, my_c, j + u, G);
            }
#pragma unroll
            for (int u = 0; u < UU; ++u)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int v = gl + r * G;
                    b[u][r] = (cc[u] >= 0 && v < nvec) ? ld_row<NC>(Bv + (long long)cc[u] * ldb_v + v) : vzero((V*)nullptr);
                }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                if (rr[u] >= 0 && rr[u] != cur_row) {
                    cur_row = rr[u];
                    const V* ap = arows.resolve(cur_row);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const int v = gl + r * G;
                        a[r] = v < nvec ? ld_row<NC>(ap + v) : vzero((V*)nullptr);
                    }
                }
                T d = 0;
#pragma unroll
                for (int r = 0; r < R; ++r) d += vdot(a[r], b[u][r]);
                acc[u] = d;
            }
            // UU dot products reduced together; value u ends up in lanes [u*G/UU, (u+1)*G/UU)
            group_transpose_reduce<T, G, UU>(acc, gmask, gl);
            const T mine = __shfl_sync(gmask, acc[0], (gl % UU) * (G / UU), G);
            if (gl / UU == j / UU) my_out = mine;  // lane gl keeps nonzero gl of the batch
        }
        if (ok) store(i, my_out);
    }
}

// ---------------------------------------------------------------------------
// SpMM
// ---------------------------------------------------------------------------
constexpr int SPMM_PIECE_SHIFT = 20;   // at most 2^20 split rows, 2^11 pieces per row

struct SpmmLong {
    const int* first_piece;  // [nlong] first carry slot of each long row
    const int* npieces;      // [nlong]
    int* counters;           // [nlong] zero at launch; reset by the finishing warp
    void* carry;             // [total pieces, ldc] scratch
    long long ldc;           // elements per carry row
    int piece_len;           // largest number of nonzeros of a piece
    int* ticket;             // optional work counter (zero at launch): items are then handed out dynamically
};

template <typename T> struct EmitLocal {
    using V = typename Vec<T>::type;
    V* Yv;
    long long ldy_v;
    T beta;
    // writes vector v of row `row`
    __device__ __forceinline__ void operator()(int row, int v, const V& acc) const {
        V* y = Yv + (long long)row * ldy_v + v;
        if (beta != (T)0) { V o = vscale(beta, *y); vadd(o, acc); *y = o; }
        else *y = acc;
    }
};

// Adds val[q] * X[colidx[q]] for q in [p0, p1) taken in batches of G (one
// coalesced index/value load per batch, broadcast inside the lane group);
// consecutive batches of this group are `batch_stride` apart.
template <typename T, int G, int R, int U, bool NC = true>
__device__ __forceinline__ void spmm_accumulate(typename Vec<T>::type (&acc)[R], long long p0, long long p1,
                                                int batch_stride, unsigned gmask,
                                                const int* __restrict__ colidx, const T* __restrict__ val,
                                                const typename Vec<T>::type* __restrict__ Xv, long long ldx_v,
                                                int gl, int nvec) {
    using V = typename Vec<T>::type;
    constexpr int UU = U < G ? U : G;
    for (long long base = p0; base < p1; base += batch_stride) {
        const long long q = base + gl;
        const bool ok = q < p1;
        const int my_c = ok ? __ldg(colidx + q) : -1;
        const T my_v = ok ? __ldg(val + q) : (T)0;
        const int n = (p1 - base) < G ? (int)(p1 - base) : G;
        for (int j = 0; j < n; j += UU) {
            int cc[UU];
            T vv[UU];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                cc[u] = __shfl_sync(gmask, my_c, j + u, G);
                vv[u] = __shfl_sync(gmask, my_v, j + u, G);
            }
            V x[UU][R];
#pragma unroll
            for (int u = 0; u < UU; ++u)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int v = gl + r * G;
                    x[u][r] = (cc[u] >= 0 && v < nvec) ? ld_row<NC>(Xv + (long long)cc[u] * ldx_v + v) : vzero((V*)nullptr);
                }
#pragma unroll
            for (int u = 0; u < UU; ++u)
#pragma unroll
                for (int r = 0; r < R; ++r) vfma(acc[r], vv[u], x[u][r]);
        }
    }
}

// Rows [r0, r1) of the CSR matrix as one flat stream of nonzeros: entries are
// fetched G at a time (the next batch is requested before the current one is
// consumed), U dense rows are in flight per lane, and the accumulator is
// emitted whenever the stream crosses into the next row.  Rows without
// nonzeros are emitted too (as zeros).  One lane group runs this alone, so no
// atomics are involved and the result is reproducible.
template <typename T, int G, int R, int U, typename Emit, bool NC = true>
__device__ __forceinline__ void spmm_rows_stream(int r0, int r1, const long long* __restrict__ rowptr,
                                                 const int* __restrict__ colidx, const T* __restrict__ val,
                                                 const typename Vec<T>::type* __restrict__ Xv, long long ldx_v,
                                                 const Emit& emit, unsigned gmask, int gl, int nvec) {
    using V = typename Vec<T>::type;
    constexpr int UU = U < G ? U : G;
    if (r0 >= r1) return;
    // positions are kept as 32-bit offsets from the first nonzero of the range (an item holds far fewer
    // than 2^31 nonzeros); the dense-row stride is a 32-bit factor so that a row address costs one wide multiply
    const long long q0 = rowptr[r0];
    const int* __restrict__ cix = colidx + q0;
    const T* __restrict__ vls = val + q0;
    const int qend = (int)(rowptr[r1] - q0);
    const int ld = (int)ldx_v;
    int base = 0;
    int row = r0;
    int row_end = (int)(rowptr[r0 + 1] - q0);
    V acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = vzero((V*)nullptr);
    auto flush = [&](int rw) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int v = gl + r * G;
            if (v < nvec) emit(rw, v, acc[r]);
            acc[r] = vzero((V*)nullptr);
        }
    };
    int nxt_c = (gl < qend) ? __ldg(cix + gl) : -1;
    T nxt_v = (gl < qend) ? __ldg(vls + gl) : (T)0;
    while (base < qend) {
        const int my_c = nxt_c;
        const T my_v = nxt_v;
        const int nb = base + G;
        nxt_c = (nb + gl < qend) ? __ldg(cix + nb + gl) : -1;
        nxt_v = (nb + gl < qend) ? __ldg(vls + nb + gl) : (T)0;
        const int n = (qend - base) < G ? (qend - base) : G;
        for (int j = 0; j < n; j += UU) {
            int cc[UU];
            T vv[UU];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                cc[u] = __shfl_sync(gmask, my_c, j + u, G);  // -1 past the end of the range
                vv[u] = __shfl_sync(gmask, my_v, j + u, G);
            }
            V x[UU][R];
#pragma unroll
            for (int u = 0; u < UU; ++u)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int v = gl + r * G;
                    x[u][r] = (cc[u] >= 0 && v < nvec) ? ld_row<NC>(Xv + (long long)cc[u] * ld + v) : vzero((V*)nullptr);
                }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                if (cc[u] >= 0) {
                    const int q = base + j + u;
                    while (q >= row_end) {
                        flush(row);
                        ++row;
                        row_end = (int)(rowptr[row + 1] - q0);
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) vfma(acc[r], vv[u], x[u][r]);
                }
            }
        }
        base = nb;
    }
    while (row < r1) {
        flush(row);
        ++row;
    }
}

template <typename T, int G, int R, int U, typename Emit, bool NC = true>
__device__ __forceinline__ void spmm_warp_item(const int4 item, const long long* __restrict__ rowptr,
                                               const int* __restrict__ colidx, const T* __restrict__ val,
                                               const typename Vec<T>::type* __restrict__ Xv, long long ldx_v,
                                               int nvec, const Emit& emit, const SpmmLong& lg, int lane) {
    using V = typename Vec<T>::type;
    constexpr int SLOTS = 32 / G;
    const int slot = lane / G, gl = lane % G;
    const unsigned gmask = group_mask<G>(slot);
    if (item.w < 0) {
        const int nr = item.y - item.x;
        const int r0 = item.x + (int)(((long long)nr * slot) / SLOTS);
        const int r1 = item.x + (int)(((long long)nr * (slot + 1)) / SLOTS);
        spmm_rows_stream<T, G, R, U, Emit, NC>(r0, r1, rowptr, colidx, val, Xv, ldx_v, emit, gmask, gl, nvec);
        return;
    }
    // piece of a long row: the warp reads 32 consecutive entries per step, each
    // group takes its G of them; groups are combined afterwards
    V acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = vzero((V*)nullptr);
    spmm_accumulate<T, G, R, U, NC>(acc, (long long)item.y + slot * G, item.z, 32, gmask, colidx, val, Xv, ldx_v, gl, nvec);
#pragma unroll
    for (int m = G; m < 32; m <<= 1)
#pragma unroll
        for (int r = 0; r < R; ++r) vadd(acc[r], shfl_xor_vec(acc[r], m));
    // item.w = long-row slot | number of this piece inside its row << SPMM_PIECE_SHIFT
    const int lr = item.w & ((1 << SPMM_PIECE_SHIFT) - 1), row = item.x;
    const int first = __ldg(lg.first_piece + lr), np = __ldg(lg.npieces + lr);
    const int piece = first + (item.w >> SPMM_PIECE_SHIFT);
    V* carry = reinterpret_cast<V*>(lg.carry);
    const long long ldc_v = lg.ldc / Vec<T>::N;
    if (slot == 0)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int v = gl + r * G;
            if (v < nvec) __stcg(carry + (long long)piece * ldc_v + v, acc[r]);
        }
    __threadfence();
    __syncwarp();
    int old = 0;
    if (lane == 0) old = atomicAdd(lg.counters + lr, 1);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != np - 1) return;
    __threadfence();
    if (slot == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int v = gl + r * G;
            if (v >= nvec) continue;
            V s = vzero((V*)nullptr);
            for (int j = 0; j < np; ++j) vadd(s, __ldcg(carry + (long long)(first + j) * ldc_v + v));
            emit(row, v, s);
        }
    }
    if (lane == 0) lg.counters[lr] = 0;
}

// Work items per ticket of a dynamically scheduled kernel: about 1/32 of a warp's share, at most max_per.
__device__ __forceinline__ int per_ticket(long long n_work, int nwarps, int max_per) {
    const long long p = n_work / ((long long)nwarps * 32);
    return p < 1 ? 1 : (p > max_per ? max_per : (int)p);
}

// ---- launch helpers ----------------------------------------------------------
inline int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

// Resident blocks of `threads` threads for a persistent launch of `kernel`.
template <typename K>
unsigned persistent_blocks(K kernel, long long needed, int threads = 256, size_t smem = 0) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
    static const int mult = env_int("SP3_PERSIST", 1);
    long long b = mult > 0 ? (long long)sms * (per_sm > 0 ? per_sm : 1) * mult : needed;
    if (needed > 0 && b > needed) b = needed;
    return (unsigned)(b > 0 ? b : 1);
}

// Lane-group shape for a row of `nvec` 16-byte vectors.  SDDMM (spmm ==
// false) runs best with about 16 lanes per row and 2-4 vectors per lane; SpMM
// with as many lanes per row as the row has vectors (measured on B200, R-MAT
// scale 20, k = 32..256).  SP3_VEC_PER_LANE overrides R for tuning.
inline void pick_shape(int nvec, int* G, int* R, bool spmm) {
    static const int forced_sddmm = env_int("SP3_VEC_PER_LANE", 0);
    static const int forced_spmm = env_int("SP3_SPMM_VEC_PER_LANE", 0);
    const int forced = spmm ? forced_spmm : forced_sddmm;
    int r = 1;
    if (!spmm) { r = 2; while (nvec > 16 * r && r < 8) r <<= 1; }
    if (forced > 0) r = forced;
    while (r > 1 && r > nvec) r >>= 1;
    int g = pick_group((nvec + r - 1) / r);
    while (g * r < nvec) r <<= 1;  // nvec > 32 * r
    *G = g; *R = r;
}

#define SP3_DISPATCH_GR(MACRO)                                                          \
    switch (R) {                                                                        \
        case 1: switch (G) { case 1: MACRO(1, 1); break; case 2: MACRO(2, 1); break; case 4: MACRO(4, 1); break; \
                             case 8: MACRO(8, 1); break; case 16: MACRO(16, 1); break; default: MACRO(32, 1); } break; \
        case 2: switch (G) { case 1: MACRO(1, 2); break; case 2: MACRO(2, 2); break; case 4: MACRO(4, 2); break; \
                             case 8: MACRO(8, 2); break; case 16: MACRO(16, 2); break; default: MACRO(32, 2); } break; \
        case 4: switch (G) { case 1: MACRO(1, 4); break; case 2: MACRO(2, 4); break; case 4: MACRO(4, 4); break; \
                             case 8: MACRO(8, 4); break; case 16: MACRO(16, 4); break; default: MACRO(32, 4); } break; \
        default: switch (G) { case 1: MACRO(1, 8); break; case 2: MACRO(2, 8); break; case 4: MACRO(4, 8); break; \
                              case 8: MACRO(8, 8); break; case 16: MACRO(16, 8); break; default: MACRO(32, 8); } break; \
    }

}  // namespace sp3

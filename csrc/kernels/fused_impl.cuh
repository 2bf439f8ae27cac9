// Fused compute + communication kernels for sm_100a, written once for both value types: this file is included
// by fused_ops.cu (fp32) and fused_ops_f64.cu (fp64) with SP3_FUSED_T, SP3_FUSED_NS, SP3_FUSED_SUFFIX and
// SP3_FUSED_IS_F32 set; everything lives in a namespace of its own per type.
//
// One persistent kernel per distributed op.  Instead of "pack, message, unpack,
// compute, message, add" (the reference's phased pipelines,
// src/distributed_comp.cpp:17-76 for SpMM and :141-284 for SDDMM, with the
// staging copies of src/comm.hpp:90-103,166-189), every rank's kernel
//
//   * pulls the dense rows it needs (B and, staged, A rows for SDDMM; X rows
//     for SpMM) straight out of the owners' memory over NVLink into its local
//     block: the first warp of every block issues one `cp.async.bulk` copy per
//     row into a shared-memory ring and one bulk store per filled stage, so no
//     compute warp ever waits for a remote load (a form with vector loads by
//     the pulling warps is kept as an option, as is reading remote A rows in
//     place through peer references);
//   * computes wave by wave: the pull tickets are grouped into a few waves
//     with one completion counter each, the work (nonzeros for SDDMM, items
//     and pieces of hub rows for SpMM) is sorted by the wave that completes
//     it, and a work ticket waits only for the waves it needs;
//   * SDDMM: keeps its partial dot products in a local array in compute order
//     and sends the ranges that belong to other fiber ranks as contiguous
//     remote stores right after each ticket; each rank then sums the Z partial
//     vectors of its own slice (the reduce-scatter of src/denseComm.hpp:35-40
//     becomes remote stores + a local sum, or one `multimem.ld_reduce` per 16
//     bytes where the fiber is bound to a multicast object);
//   * SpMM: stores finished partial rows of rows it does not own directly into
//     a slot in the owner's memory; the owner adds its own partial and the
//     slots in ascending source order (bitwise reproducible), which is the
//     role-swapped exchange + SUM_from_recvbuff of src/comm.hpp:178-189.
//
// Moved data is exactly what the plan lists (the sparsity-aware minimum).
//
// Cross-GPU ordering uses three flags per (source rank, kind) in a signal pad
// in every rank's symmetric heap, written with st.release.sys and read with
// ld.acquire.sys, carrying the epoch (launch number) of the op:
//   READY  "my operands for this epoch may be read"      -> my readers
//   DONE   "I no longer read your memory this epoch"      -> ranks I read from
//   PART   "my partial results for this epoch are in your memory" -> targets
// A kernel returns only after every rank that reads its memory has signalled
// DONE, so when the op completes the caller may overwrite its operands.
// Partial-result buffers are double buffered by epoch parity.  Every wait is
// bounded: on timeout the kernel records {code, site, peer, value} in the
// status words, raises the abort flag so the other warps drain, and returns.
//
// The three phases (START = publish READY, MAIN = pull + compute + push,
// FINISH = reduce + final handshake) run in one launch; they can also be
// launched one at a time, which lets a single GPU run all ranks of a mesh in
// lock step (each phase of every rank before the next phase) without any
// kernel ever waiting on a later launch.
#pragma once
#include "sp3_kernels.cuh"
#include "sp3_async.cuh"


namespace sp3 {
namespace SP3_FUSED_NS {

using real = SP3_FUSED_T;           // value type of this instantiation of the file
using vec = Vec<real>::type;        // 16-byte vector of values
constexpr int VN = Vec<real>::N;    // values per vector
constexpr bool IS_F32 = sizeof(real) == 4;

constexpr int MAX_RANKS = 64;
enum FlagKind : int { F_READY = 0, F_DONE = 1, F_PART = 2, F_KINDS = 3 };
constexpr int MAX_WAVES = 32;
// words [C_WAVE0, C_WAVE0 + MAX_WAVES): pull tiles finished per wave (see FusedSddmmArgs::wave_nnz)
enum Ctrl : int { C_TICKET_MAIN = 0, C_PULLS_DONE = 1, C_MAIN_DONE = 2, C_TICKET_FIN = 3, C_FIN_DONE = 4, C_ABORT = 5, C_TICKET_WORK = 6, C_WORK_DONE = 7, C_TICKET_PUSH = 8, C_TICKET_START = 9, C_START_DONE = 10, C_WAVE0 = 16, C_WORDS = C_WAVE0 + MAX_WAVES };
enum Phase : int { PH_START = 1, PH_MAIN = 2, PH_FINISH = 4 };
enum WaitSite : int { W_READY = 1, W_PULLS = 2, W_PART = 3, W_DONE = 4, W_WORK = 5 };

constexpr int REDUCE_ELEMS = 2048; // values per SDDMM reduce ticket
constexpr int PUSH_ELEMS = 4096;   // partial values per SDDMM push ticket
constexpr int REDUCE_ROWS = 32;    // owned rows per SpMM reduce ticket

struct FusedComm {
    int me;                  // my world rank
    int epoch;               // launch number of this op, >= 1
    int phases;              // Phase bits
    unsigned long long timeout_ns;
    int* status;             // int[4] local
    int* ctrl;               // int[C_WORDS] local, zero at launch
    int* pad;                // my signal pad, int[F_KINDS][MAX_RANKS], indexed by source rank
    int* const* peer_pad;    // [world] every rank's pad as mapped into this process
    const int* read_from;    // ranks whose memory I read
    const int* readers;      // ranks that read my memory
    const int* push_to;      // ranks I push partial results to
    const int* contrib;      // ranks that push partial results to me
    int n_read, n_readers, n_push, n_contrib;
    unsigned long long* stamps;  // optional [4]: globaltimer at kernel start, last pull done, MAIN done, FINISH done
};

enum Stamp : int { T_START = 0, T_PULLED = 1, T_MAIN = 2, T_FINISH = 3 };
__device__ __forceinline__ void stamp(const FusedComm& c, int which) {
    if (c.stamps) c.stamps[which] = globaltimer_ns();
}

// Work is handed out by one counter; a ticket covers `n` consecutive work
// items so that the counter sees a few ten-thousand atomics per launch instead
// of one per item (atomics on one address serialise in L2).
__device__ __forceinline__ int warp_ticket(int* ctr, int lane, int n = 1) {
    int t = 0;
    if (lane == 0) t = atomicAdd(ctr, n);
    return __shfl_sync(0xffffffffu, t, 0);
}

// Work per ticket: large enough to keep the counter quiet, small enough that the last tickets (the tail of
// the kernel, when other warps already idle) are short: about 1/32 of a warp's share, at most MAX.
constexpr int SDDMM_UNITS_PER_TICKET_MAX = 8;
constexpr int SPMM_ITEMS_PER_TICKET_MAX = 4;


__device__ __forceinline__ bool aborted(const FusedComm& c) {
    return *reinterpret_cast<volatile int*>(c.ctrl + C_ABORT) != 0;
}

__device__ __forceinline__ void signal(const FusedComm& c, int kind, int dst) {
    st_release_sys(c.peer_pad[dst] + kind * MAX_RANKS + c.me, c.epoch);
}

// Bounded wait for flag[kind][src] >= epoch.  All lanes may call it; they all
// poll (reads of one word).  On timeout: status record + abort flag.
__device__ __forceinline__ bool wait_flag(const FusedComm& c, int kind, int src, int site) {
    const int* f = c.pad + kind * MAX_RANKS + src;
    if (ld_acquire_sys(f) >= c.epoch) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i) {
            if (ld_acquire_sys(f) >= c.epoch) return true;
            __nanosleep(100);
        }
        if (aborted(c)) return false;
        if (globaltimer_ns() - t0 > c.timeout_ns) {
            report(c.status, ST_WAIT_TIMEOUT, site, src, ld_acquire_sys(f));
            atomicExch(c.ctrl + C_ABORT, 1);
            return false;
        }
    }
}

__device__ __forceinline__ bool wait_all(const FusedComm& c, int kind, const int* list, int n, int site) {
    bool ok = true;
    for (int i = 0; i < n; ++i) ok = wait_flag(c, kind, list[i], site) && ok;
    return ok;
}

__device__ __forceinline__ bool wait_counter(const FusedComm& c, int which, int want, int site) {
    const int* p = c.ctrl + which;
    if (ld_acquire_gpu(p) >= want) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i) {
            if (ld_acquire_gpu(p) >= want) return true;
            __nanosleep(64);
        }
        if (aborted(c)) return false;
        if (globaltimer_ns() - t0 > c.timeout_ns) {
            report(c.status, ST_WAIT_TIMEOUT, site, which, ld_acquire_gpu(p));
            atomicExch(c.ctrl + C_ABORT, 1);
            return false;
        }
    }
}

__device__ __forceinline__ void start_phase(const FusedComm& c) {
    if (blockIdx.x == 0 && threadIdx.x == 0) stamp(c, T_START);
    if (blockIdx.x == 0 && threadIdx.x < c.n_readers) {
        __threadfence_system();
        signal(c, F_READY, c.readers[threadIdx.x]);
    }
}

// Copies dense rows [r0, r1) of a receive list from their owners' memory
// (src[r] = absolute address of the row, local or peer) into the local block.
// The tile is treated as a flat list of 16-byte vectors, eight per lane in
// flight, so a warp keeps 4 KB of NVLink reads outstanding.
__device__ __forceinline__ void pull_rows(int r0, int r1, const float4* const* __restrict__ src,
                                          float4* __restrict__ dst, long long ld_v, int nvec, int lane) {
    const int total = (r1 - r0) * nvec;
    constexpr int PU = 8;
    for (int base = 0; base < total; base += 32 * PU) {
        float4 v[PU];
        int row[PU], vec[PU];
#pragma unroll
        for (int u = 0; u < PU; ++u) {
            const int e = base + u * 32 + lane;
            row[u] = e < total ? e / nvec : -1;
            vec[u] = e - row[u] * nvec;
        }
#pragma unroll
        for (int u = 0; u < PU; ++u)
            if (row[u] >= 0) v[u] = __ldcs(ldg_ptr(src + r0 + row[u]) + vec[u]);
#pragma unroll
        for (int u = 0; u < PU; ++u)
            if (row[u] >= 0) dst[(long long)(r0 + row[u]) * ld_v + vec[u]] = v[u];
    }
}

// The same copy with the asynchronous copy unit (bulk mode): one warp per block keeps a ring of BULK_STAGES
// shared-memory stages; every dense row travels as one `cp.async.bulk` load from its owner's memory (a peer
// mapping or local) into a stage, completing on the stage's mbarrier, and every filled stage leaves as one bulk
// store into the local block (the rows of a tile are consecutive there).  Nothing passes through registers and
// the warp never stalls on a load, so a few warps keep NVLink busy while all the others compute.
constexpr int BULK_STAGES = 3;
constexpr int BULK_MAX_PULLERS = 4;   // puller warps per block

// Pull set-up of a launch (host side -> kernel): how many warps of every block pull with bulk copies (0: vector
// loads), the bytes of one ring stage and the dense rows of one pull ticket.
struct PullConfig {
    int pullers;
    unsigned stage_bytes;
    int tile_rows;
};
inline size_t bulk_smem_bytes(const PullConfig& pc) {
    return pc.pullers > 0 ? (size_t)pc.pullers * BULK_STAGES * (pc.stage_bytes + 8) + 64 : 0;
}

struct BulkRing {
    unsigned ring, bars;    // shared-memory addresses of this warp's stages and of their mbarriers
    unsigned stage_bytes;
    unsigned long long g;   // chunks this warp has issued so far: stage g % BULK_STAGES, phase parity (g / BULK_STAGES) & 1
};

// Ring of puller warp `w` of this block inside the dynamic shared memory; warp w initialises its own barriers.
__device__ __forceinline__ BulkRing bulk_ring_init(unsigned char* dyn_smem, const PullConfig& pc, int warp, int lane) {
    BulkRing br{0u, 0u, pc.stage_bytes, 0ull};
    if (pc.pullers <= 0) return br;
    const unsigned base = smem_u32(dyn_smem);
    br.ring = base + (unsigned)warp * BULK_STAGES * pc.stage_bytes;
    br.bars = base + (unsigned)pc.pullers * BULK_STAGES * pc.stage_bytes + (unsigned)warp * BULK_STAGES * 8u;
    if (warp < pc.pullers && lane == 0) {
        for (int st = 0; st < BULK_STAGES; ++st) mbar_init(br.bars + 8u * st, 1);
        mbar_init_fence();
    }
    return br;
}

// Copies rows [r0, r1) of a receive list into dst (row r lands at dst + r * nvec vectors; the local block has
// no padding between rows).  All lanes of one warp call it.  Returns false when a load did not arrive in time
// (status recorded, abort raised); the copies still in flight are then given the same time again before the
// warp moves on, because their destination is this block's shared memory.
//
// drain = true: returns when the stores of this tile are complete.  drain = false: returns as soon as the last
// store is issued, so that the next tile's loads start without a pipeline bubble; `after_first_store` is called
// once the first store group of this tile is committed and all older groups (the previous tile's stores) are
// complete -- the place to publish the previous tile.  The caller publishes the last tile after bulk_drain().
// Until all bulk stores of this warp are complete and ordered before the ordinary accesses that publish them.
__device__ __forceinline__ void bulk_drain(int lane) {
    if (lane == 0) {
        bulk_wait<0>();
        fence_async_proxy();
    }
    __syncwarp();
}

template <typename F>
__device__ __forceinline__ bool bulk_pull_tile(BulkRing& br, const FusedComm& c, int r0, int r1,
                                               const float4* const* __restrict__ src, float4* __restrict__ dst,
                                               int nvec, int lane, bool drain, F&& after_first_store) {
    const unsigned row_bytes = (unsigned)nvec * 16u;
    int rps = (int)(br.stage_bytes / row_bytes);   // rows per stage
    rps = rps < 1 ? 1 : rps;
    const int n = r1 - r0, nch = (n + rps - 1) / rps;
    bool ok = true;
    for (int ch = 0; ch < nch + BULK_STAGES - 1; ++ch) {
        if (ch < nch && ok) {
            const unsigned st = (unsigned)((br.g + ch) % BULK_STAGES);
            // the store that read this stage last was issued one step ago at the latest: wait until it has let go
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
            const int c0 = ch * rps, cn = n - c0 < rps ? n - c0 : rps;
            if (lane == 0) mbar_expect_tx(br.bars + 8u * st, (unsigned)cn * row_bytes);
            __syncwarp();
            for (int i = lane; i < cn; i += 32)
                bulk_load(br.ring + st * br.stage_bytes + (unsigned)i * row_bytes, ldg_ptr(src + r0 + c0 + i),
                          row_bytes, br.bars + 8u * st);
        }
        const int pc = ch - (BULK_STAGES - 1);
        if (pc >= 0 && pc < nch) {
            const unsigned long long gi = br.g + pc;
            const unsigned st = (unsigned)(gi % BULK_STAGES), par = (unsigned)((gi / BULK_STAGES) & 1);
            const bool arrived = mbar_wait_ns(br.bars + 8u * st, par, c.timeout_ns);
            if (!arrived && ok) {
                ok = false;
                report(c.status, ST_WAIT_TIMEOUT, W_PULLS, r0 + pc * rps, (int)st);
                atomicExch(c.ctrl + C_ABORT, 1);
            }
            if (ok) {
                const int c0 = pc * rps, cn = n - c0 < rps ? n - c0 : rps;
                if (lane == 0) {
                    bulk_store(dst + (long long)(r0 + c0) * nvec, br.ring + st * br.stage_bytes, (unsigned)cn * row_bytes);
                    bulk_commit();
                }
                if (pc == 0 && !drain) {
                    if (lane == 0) {
                        bulk_wait<1>();        // every group but the one just committed: the previous tile is complete
                        fence_async_proxy();
                    }
                    __syncwarp();
                    after_first_store();
                }
            }
        }
    }
    br.g += nch;
    if (drain) bulk_drain(lane);
    return ok;
}

// ---------------------------------------------------------------------------
// Pulls and their waves, shared by both kernels.  The functions are deliberately not inlined: they run once per
// pull ticket or per work ticket, and inlined into the kernels their state takes registers from the inner loops.
// ---------------------------------------------------------------------------
struct PullSide {
    const float4* const* src;   // absolute address of every row of the receive list
    float4* dst;                // where row 0 of the list lands; rows are `ld_v` vectors apart
    int n_rows;
};

struct PullGate {
    FusedComm c;                // a copy: pointing into the kernel's parameters would move all of them to local memory
    PullSide side[2];           // SDDMM: [0] = B rows, [1] = staged A rows; SpMM: [0] = X rows
    const int* order;           // ticket -> side << 30 | tile (null: all tiles of side 1, then side 0)
    const long long* limit;     // shared memory: work runnable once the first w waves are complete, w = 0 .. n_waves
    long long ld_v;
    int nvec, tile_rows, n_pull, tiles1, tpw, n_waves;
    bool bulk, pulls_left;
    int waves_ready;            // leading waves this warp knows to be complete
    int pending;                // bulk mode: ticket whose stores are issued but not yet published (-1: none)
    BulkRing br;

    // Tells the other warps that the rows of ticket t are in the local block.
    __device__ __forceinline__ void publish(int t, int lane) {
        __threadfence();
        __syncwarp();
        if (lane == 0) {
            atomicAdd(c.ctrl + C_WAVE0 + t / tpw, 1);
            if (atomicAdd(c.ctrl + C_PULLS_DONE, 1) == n_pull - 1) stamp(c, T_PULLED);
        }
    }
    // Publishes the tile that is still in flight (bulk mode); before this warp waits for anybody or leaves.
    __device__ __forceinline__ void flush(int lane) {
        if (pending >= 0) {
            bulk_drain(lane);
            publish(pending, lane);
            pending = -1;
        }
    }
    // Serves one pull ticket; false when none is left (or a bulk copy timed out).  In bulk mode the tile is
    // published when the next one is under way (or by flush), so that the copies of consecutive tiles overlap.
    __device__ __noinline__ bool pull_one(int lane) {
        const int t = warp_ticket(c.ctrl + C_TICKET_MAIN, lane);
        if (t >= n_pull) { flush(lane); return false; }
        const int code = order ? __ldg(order + t) : (t < tiles1 ? (t | (1 << 30)) : t - tiles1);
        const int tile = code & ((1 << 30) - 1);
        const PullSide& sd = side[code >> 30];
        const int r0 = tile * tile_rows;
        const int r1 = r0 + tile_rows < sd.n_rows ? r0 + tile_rows : sd.n_rows;
        if (bulk) {
            const bool ok = bulk_pull_tile(br, c, r0, r1, sd.src, sd.dst, nvec, lane, false, [&]() {
                if (pending >= 0) { publish(pending, lane); pending = -1; }
            });
            if (!ok) { bulk_drain(lane); pending = -1; return false; }
            pending = t;
            return true;
        }
        pull_rows(r0, r1, sd.src, sd.dst, ld_v, nvec, lane);
        publish(t, lane);
        return true;
    }
    __device__ __noinline__ void pull_all(int lane) {
        while (pulls_left && !aborted(c)) pulls_left = pull_one(lane);
        flush(lane);
    }
    // Makes sure that every wave the work below `upto` needs is complete: a warp whose work is not ready serves a
    // pull ticket (vector-load mode; every ticket is thus taken by a running warp and the wait cannot deadlock)
    // and looks again; when no ticket is left for it, it waits, with a time limit, for the warps that still copy.
    __device__ __noinline__ bool ensure_slow(long long upto, int lane) {
        while (waves_ready < n_waves && upto > limit[waves_ready]) {
            const int w = waves_ready;
            const int want = (w + 1) * tpw <= n_pull ? tpw : n_pull - w * tpw;
            if (ld_acquire_gpu(c.ctrl + C_WAVE0 + w) >= want) { ++waves_ready; continue; }
            if (pulls_left) { pulls_left = pull_one(lane); continue; }
            flush(lane);   // never wait while a tile of this warp is unpublished
            if (!wait_counter(c, C_WAVE0 + w, want, W_PULLS)) return false;
            ++waves_ready;
        }
        return true;
    }
    __device__ __forceinline__ bool ensure(long long upto, int lane) {
        if (waves_ready >= n_waves || upto <= limit[waves_ready]) return true;
        return ensure_slow(upto, lane);
    }
};

// Every warp calls this after its MAIN work; the last one to arrive publishes
// DONE and PART for this rank.
__device__ __forceinline__ void main_epilogue(const FusedComm& c, int lane, int nwarps) {
    // remote stores (pushed partial results) must be visible system-wide before PART is signalled; a rank
    // that pushed nothing only has to order its local writes
#ifndef SP3_EPILOGUE_GPU_FENCE
    if (c.n_push > 0) __threadfence_system();
    else __threadfence();
#else
    __threadfence();
#endif
    __syncwarp();
    int old = 0;
    if (lane == 0) old = atomicAdd(c.ctrl + C_MAIN_DONE, 1);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old == nwarps - 1) {
        __threadfence_system();
        for (int i = lane; i < c.n_read; i += 32) signal(c, F_DONE, c.read_from[i]);
        for (int i = lane; i < c.n_push; i += 32) signal(c, F_PART, c.push_to[i]);
        if (lane == 0) stamp(c, T_MAIN);
    }
}

// Last warp of the FINISH phase keeps the kernel alive until every reader of
// this rank's memory is done with it.
__device__ __forceinline__ void finish_epilogue(const FusedComm& c, int lane, int nwarps) {
    __syncwarp();
    int old = 0;
    if (lane == 0) old = atomicAdd(c.ctrl + C_FIN_DONE, 1);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old == nwarps - 1 && lane == 0) {
        wait_all(c, F_DONE, c.readers, c.n_readers, W_DONE);
        stamp(c, T_FINISH);
    }
}

// ---------------------------------------------------------------------------
// SDDMM
// ---------------------------------------------------------------------------
struct FusedSddmmArgs {
    FusedComm comm;
    long long nnz;
    const int* rowidx;
    const int* colidx;
    const real* sval;
    const int* a_refs;            // [rows of the local A layout] owner rank << 25 | row in the owner's block;
                                  // null when the needed remote rows are staged (every row is then local)
    const unsigned long long* a_bases;  // [world] address of every rank's A block as mapped here
    int world;
    real* B_loc;                 // local B block [owned | pulled]
    long long ldb;
    int n_owned_b, n_recv_b;
    const float4* const* b_src;   // [n_recv_b] absolute addresses of the rows to pull
    int nvec;
    int Z, my_z;
    unsigned zbase, zrem;         // slice lengths: zbase (+1 for the first zrem fiber ranks)
    long long zwidth;             // elements reserved per (parity, source) in a value buffer
    real* const* zbuf;           // [Z] value buffers of the fiber ranks (mine is local)
    real* out;                   // my slice of C
    real* part;                  // [nnz] local partial values (used when Z > 1)
    int direct_push;              // 1: values of other fiber ranks are stored remotely as they are computed;
                                  // 0: they are staged in `part` and pushed in bulk once all are there;
                                  // 2: staged, and every warp pushes the range of a ticket right after computing
                                  //    it (needs orig == null: a ticket's values are then one contiguous range)
                                  // 3: staged in a multicast-bound buffer, nothing pushed, reduced in the switch
    // Overlap of pulls and compute: the kernel walks the nonzeros in the order "those whose B row is owned
    // first, then those that need a pulled row" (rowidx / colidx / sval are given in that order);
    // orig[i] is the position of nonzero i in the plan's value order (null: identity), nnz_free the
    // length of the first part, work_per_pull how many compute tickets a warp takes per pull ticket.
    const int* orig;
    long long nnz_free;
    int work_per_pull;
    // Staging of remote A rows (optional; n_recv_a == 0: A rows are read in place from their owners): the needed
    // rows a_src[0..n_recv_a) are pulled to A_stage, which follows my owned rows in my own A block.
    int n_recv_a;
    const float4* const* a_src;
    real* A_stage;
    // Z reduction inside the NVSwitch (direct_push == 3): `part` is this rank's buffer of a symmetric allocation
    // that is bound to a multicast object over the Z fiber ([2][part_stride] values, one half per epoch parity);
    // nothing is pushed, and in FINISH the owner of a slice reads mc_part (the multicast address of the same
    // allocation) with `multimem.ld_reduce.add`, which returns the sum over all fiber ranks.
    const real* mc_part;
    long long part_stride;
    // Pull waves.  The pull tickets are served in the order pull_order[t] (bit 30 set: tile of needed A rows,
    // else tile of needed B rows; low bits: tile number; null: A tiles then B tiles) and grouped into n_waves
    // waves of tiles_per_wave consecutive tickets.  The nonzeros are given sorted by the last wave that brings
    // one of their two rows (class 0: both rows owned); wave_nnz[c] (c = 0..n_waves) is the number of nonzeros
    // that can be computed once the first c waves are complete.  A work unit waits only for the waves its own
    // nonzeros need, so compute follows the pulls wave by wave instead of starting after the last tile.
    const int* pull_order;
    int n_waves, tiles_per_wave;
    const long long* wave_nnz;
    PullConfig pull;              // who pulls, and in which portions (see PullConfig, bulk_pull_tile)
};

#if SP3_FUSED_IS_F32
// Sum over all devices of a multicast object, added in the NVSwitch (NVLS); `p` is a multicast address.
__device__ __forceinline__ float multimem_add_f32(const float* p) {
    float v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 multimem_add_v4(const float* p) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
#endif

// Adds a 16-byte vector into memory that other ranks add into as well: one vector atomic (fp32), or one
// atomic per value.
__device__ __forceinline__ void vatomic_add(vec* y, const vec& acc, bool whole_vector) {
#if SP3_FUSED_IS_F32
    if (whole_vector) { atomicAdd(y, acc); return; }
    real* f = reinterpret_cast<real*>(y);
    atomicAdd(f, acc.x); atomicAdd(f + 1, acc.y); atomicAdd(f + 2, acc.z); atomicAdd(f + 3, acc.w);
#else
    (void)whole_vector;
    real* f = reinterpret_cast<real*>(y);
    atomicAdd(f, acc.x); atomicAdd(f + 1, acc.y);
#endif
}

// Where a value goes.  Z == 1: into the result.  Z > 1, staged mode: into the local array `part` at its
// position in the plan's value order; the slices of the other fiber ranks are then pushed in bulk by the
// push tickets of the MAIN phase.  Z > 1, direct mode: values of my own slice into `part`, the others
// straight into their owner's buffer.
struct StorePartial {
    const real* sval;
    const int* orig;
    real* dst;           // local: `part` (Z > 1, staged), or the result (Z == 1)
    real* const* zbuf;   // direct mode: value buffers of the fiber ranks
    int direct, Z, my_z, parity;
    unsigned zbase, zrem;
    long long zwidth;
    __device__ __forceinline__ void operator()(long long i, real dot) const {
        const unsigned ii = orig ? (unsigned)__ldg(orig + i) : (unsigned)i;
        const real v = dot * __ldg(sval + i);
        if (!direct) { dst[ii] = v; return; }
        // direct mode (wide rows: a lane group stores >= 32 contiguous bytes): straight into the owner's buffer
        const unsigned split = zrem * (zbase + 1);
        unsigned zo, off;
        if (ii < split) { zo = ii / (zbase + 1); off = zo * (zbase + 1); }
        else { zo = zrem + (ii - split) / zbase; off = split + (zo - zrem) * zbase; }
        if ((int)zo == my_z) dst[ii] = v;
        else zbuf[zo][((long long)parity * Z + my_z) * zwidth + (ii - off)] = v;
    }
};

__device__ __forceinline__ long long slice_off(int z, unsigned zbase, unsigned zrem) {
    return (long long)z * zbase + ((unsigned)z < zrem ? z : (int)zrem);
}

template <int G, int R, int U>
__global__ void __launch_bounds__(256, sddmm_min_blocks(R)) fused_sddmm_kernel(const FusedSddmmArgs a) {
    const FusedComm& c = a.comm;
    const int lane = threadIdx.x & 31;
    const int nwarps = (int)(((long long)gridDim.x * blockDim.x) >> 5);
    const int parity = c.epoch & 1;
    __shared__ unsigned long long a_bases[MAX_RANKS];
    __shared__ long long wave_limit[MAX_WAVES + 1];
    extern __shared__ __align__(128) unsigned char dyn_smem[];   // bulk mode: the pullers' rings, else nothing
    if (threadIdx.x < MAX_RANKS) a_bases[threadIdx.x] = threadIdx.x < a.world ? a.a_bases[threadIdx.x] : 0ull;
    const bool bulk = a.pull.pullers > 0;
    const int PULL_ROWS = a.pull.tile_rows;
    BulkRing br = bulk_ring_init(dyn_smem, a.pull, threadIdx.x >> 5, lane);
    __syncthreads();
    if (c.phases & PH_START) start_phase(c);
    if (c.phases & PH_MAIN) {
        if (!(c.phases & PH_START) && blockIdx.x == 0 && threadIdx.x == 0) stamp(c, T_START);
        bool ok = wait_all(c, F_READY, c.read_from, c.n_read, W_READY);
        constexpr int SLOTS = 32 / G;
        // pull tickets: tiles of needed A rows first (when A rows are staged), then tiles of needed B rows
        const int n_pull_a = (a.n_recv_a + PULL_ROWS - 1) / PULL_ROWS;
        const int n_pull = n_pull_a + (a.n_recv_b + PULL_ROWS - 1) / PULL_ROWS;
        const long long per_unit = (long long)SLOTS * SDDMM_PER_SLOT;
        const long long n_units = (a.nnz + per_unit - 1) / per_unit;
        const RowsByPeerRef<real> arows{a.a_refs, a_bases, (unsigned long long)a.nvec * 16ull, c.me << PEER_REF_SHIFT};
        const int direct = a.Z > 1 && a.direct_push == 1;
        const bool self_push = a.Z > 1 && a.direct_push == 2 && a.orig == nullptr;
        const bool in_switch = a.Z > 1 && a.direct_push == 3;
        real* const part = in_switch ? a.part + (long long)parity * a.part_stride : a.part;
        const StorePartial store{a.sval, a.orig, a.Z > 1 ? part : a.out, a.zbuf, direct, a.Z, a.my_z, parity,
                                 a.zbase, a.zrem, a.zwidth};
        vec* Bv = reinterpret_cast<vec*>(a.B_loc);
        const long long ldb_v = a.ldb / VN;
        const long long gwarp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
        // pullers: in bulk mode the first warps of every block and nobody else; otherwise one warp in four,
        // helped by any warp whose own units are not ready yet
        const bool is_puller = bulk ? (int)(threadIdx.x >> 5) < a.pull.pullers : (gwarp & 3) == 0;
        const int n_waves = n_pull > 0 ? (a.n_waves > 0 ? a.n_waves : 1) : 0;
        // units runnable once the first w waves are complete (w = 0: the units that need no pulled row)
        if ((int)threadIdx.x <= n_waves) {
            const int w = threadIdx.x;
            const long long z = w >= n_waves ? a.nnz : (a.wave_nnz ? a.wave_nnz[w] : a.nnz_free);
            wave_limit[w] = z >= a.nnz ? n_units : z / per_unit;
        }
        __syncthreads();
        PullGate gate;
        gate.c = c;
        gate.side[0] = {a.b_src, reinterpret_cast<float4*>(Bv + (long long)a.n_owned_b * ldb_v), a.n_recv_b};
        gate.side[1] = {a.a_src, reinterpret_cast<float4*>(a.A_stage), a.n_recv_a};
        gate.order = a.pull_order;
        gate.limit = wave_limit;
        gate.ld_v = ldb_v;
        gate.nvec = a.nvec; gate.tile_rows = PULL_ROWS; gate.n_pull = n_pull; gate.tiles1 = n_pull_a;
        gate.tpw = a.n_waves > 0 ? a.tiles_per_wave : (n_pull > 0 ? n_pull : 1);
        gate.n_waves = n_waves;
        gate.bulk = bulk;
        gate.pulls_left = n_pull > 0 && (!bulk || is_puller);
        gate.waves_ready = 0;
        gate.pending = -1;
        gate.br = br;
        // The pullers serve pull tickets until none are left while the others start on the units that need no
        // pulled row.
        if (is_puller && ok) gate.pull_all(lane);
        const int SDDMM_UNITS_PER_TICKET = per_ticket(n_units, nwarps, SDDMM_UNITS_PER_TICKET_MAX);
        while (ok) {
            const long long u0 = (long long)warp_ticket(c.ctrl + C_TICKET_WORK, lane, SDDMM_UNITS_PER_TICKET);
            if (u0 >= n_units) break;
            const long long u1 = u0 + SDDMM_UNITS_PER_TICKET < n_units ? u0 + SDDMM_UNITS_PER_TICKET : n_units;
            ok = gate.ensure(u1, lane);
            if (!ok) break;
            for (long long u = u0; u < u1; ++u)
                sddmm_warp_unit<real, G, R, U, RowsByPeerRef<real>, StorePartial, false>(
                    u, a.nnz, a.rowidx, a.colidx, arows, Bv, ldb_v, a.nvec, store, lane);
            if (self_push) {
                // the values [i0, i1) of `part` were written by this warp just now (still in L2): send the pieces
                // that belong to other fiber ranks as contiguous remote stores while other warps compute
                __syncwarp();
                const long long i0 = u0 * per_unit, i1 = u1 * per_unit < a.nnz ? u1 * per_unit : a.nnz;
                for (int z = 0; z < a.Z; ++z) {
                    if (z == a.my_z) continue;
                    const long long s0 = slice_off(z, a.zbase, a.zrem);
                    const long long s1 = s0 + a.zbase + ((unsigned)z < a.zrem ? 1 : 0);
                    const long long j0 = i0 > s0 ? i0 : s0, j1 = i1 < s1 ? i1 : s1;
                    if (j0 >= j1) continue;
                    real* dst = a.zbuf[z] + ((long long)parity * a.Z + a.my_z) * a.zwidth - s0;
                    for (long long j = j0 + lane; j < j1; j += 128) {
                        real v[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) v[q] = (j + 32 * q < j1) ? __ldcg(a.part + j + 32 * q) : (real)0;
#pragma unroll
                        for (int q = 0; q < 4; ++q) if (j + 32 * q < j1) __stcs(dst + j + 32 * q, v[q]);
                    }
                }
            }
        }
        if (ok) gate.pull_all(lane);  // no compute left but tiles remain (tiny blocks)
        if (a.Z > 1 && !direct && !self_push && !in_switch) {
            // all partial values of this rank are in `part` once every warp has passed this point; then the
            // slices of the other fiber ranks travel as contiguous, fully coalesced remote stores
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(c.ctrl + C_WORK_DONE, 1);
            if (ok) ok = wait_counter(c, C_WORK_DONE, nwarps, W_WORK);
            const int cps = (int)((a.zwidth + PUSH_ELEMS - 1) / PUSH_ELEMS);
            while (ok) {
                const int t = warp_ticket(c.ctrl + C_TICKET_PUSH, lane);
                if (t >= cps * a.Z) break;
                const int z = t / cps, chunk = t % cps;
                if (z == a.my_z) continue;
                const long long len = a.zbase + ((unsigned)z < a.zrem ? 1 : 0);
                const long long j0 = (long long)chunk * PUSH_ELEMS;
                const long long j1 = j0 + PUSH_ELEMS < len ? j0 + PUSH_ELEMS : len;
                const real* src = a.part + slice_off(z, a.zbase, a.zrem);
                real* dst = a.zbuf[z] + ((long long)parity * a.Z + a.my_z) * a.zwidth;
                for (long long j = j0 + lane; j < j1; j += 128) {
                    real v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = (j + 32 * u < j1) ? __ldcg(src + j + 32 * u) : (real)0;
#pragma unroll
                    for (int u = 0; u < 4; ++u) if (j + 32 * u < j1) __stcs(dst + j + 32 * u, v[u]);
                }
            }
        }
        main_epilogue(c, lane, nwarps);
    }
    if (c.phases & PH_FINISH) {
        if (a.Z > 1) {
            bool ok = wait_all(c, F_PART, c.contrib, c.n_contrib, W_PART);
            // my own partials come from my own MAIN warps (same launch): wait for all of them
            if (ok && (c.phases & PH_MAIN)) ok = wait_counter(c, C_MAIN_DONE, nwarps, W_PART);
            const long long my_len = a.zbase + ((unsigned)a.my_z < a.zrem ? 1 : 0);
            const int n_chunks = (int)((my_len + REDUCE_ELEMS - 1) / REDUCE_ELEMS);
            const real* mine = a.zbuf[a.my_z] + (long long)parity * a.Z * a.zwidth;
            const real* own = a.part + slice_off(a.my_z, a.zbase, a.zrem);
#if SP3_FUSED_IS_F32
            while (ok && a.direct_push == 3) {
                // one load per 16 bytes returns the sum over the fiber, added inside the switch; positions of
                // the multicast buffer that are not 16-byte aligned (slice edges) are read one value at a time
                const int t = warp_ticket(c.ctrl + C_TICKET_FIN, lane);
                if (t >= n_chunks) break;
                const long long s0 = slice_off(a.my_z, a.zbase, a.zrem);
                const real* src = a.mc_part + (long long)parity * a.part_stride;   // 16-byte aligned
                const long long j0 = s0 + (long long)t * REDUCE_ELEMS;
                const long long j1 = j0 + REDUCE_ELEMS < s0 + my_len ? j0 + REDUCE_ELEMS : s0 + my_len;
                const long long b0 = (j0 + 3) & ~3ll, b1 = j1 & ~3ll;     // aligned body [b0, b1)
                if (b0 >= b1) {
                    for (long long j = j0 + lane; j < j1; j += 32) a.out[j - s0] = multimem_add_f32(src + j);
                } else {
                    for (long long j = j0 + lane; j < b0; j += 32) a.out[j - s0] = multimem_add_f32(src + j);
                    for (long long j = b0 + 4 * lane; j < b1; j += 128) {
                        const vec v = multimem_add_v4(src + j);
                        real* o = a.out + (j - s0);
                        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
                    }
                    for (long long j = b1 + lane; j < j1; j += 32) a.out[j - s0] = multimem_add_f32(src + j);
                }
            }
#endif
            while (ok && a.direct_push != 3) {
                const int t = warp_ticket(c.ctrl + C_TICKET_FIN, lane);
                if (t >= n_chunks) break;
                const long long e0 = (long long)t * REDUCE_ELEMS;
                const long long e1 = e0 + REDUCE_ELEMS < my_len ? e0 + REDUCE_ELEMS : my_len;
                // four values per lane and step, so that 4 * Z independent loads are in flight per lane
                for (long long j = e0 + lane; j < e1; j += 128) {
                    real s[4] = {(real)0, (real)0, (real)0, (real)0};  // fiber ranks in ascending order; my own partial comes from `part`
                    for (int z = 0; z < a.Z; ++z) {
                        const real* src = z == a.my_z ? own : mine + (long long)z * a.zwidth;
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (j + 32 * q < e1) s[q] += __ldcg(src + j + 32 * q);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (j + 32 * q < e1) a.out[j + 32 * q] = s[q];
                }
            }
        }
        finish_epilogue(c, lane, nwarps);
    }
}

// ---------------------------------------------------------------------------
// SpMM
// ---------------------------------------------------------------------------
struct FusedSpmmArgs {
    FusedComm comm;
    int nitems;
    const int4* items;
    const long long* rowptr;
    const int* colidx;
    const real* val;
    real* X_loc;                 // local X block [owned | pulled]
    long long ldx;
    int n_owned_x, n_recv_x;
    const float4* const* x_src;   // [n_recv_x]
    int nvec;
    SpmmLong lg;
    int n_owned_y;
    int n_crows;                  // owned rows that receive contributions from peers
    const int* crows;             // [n_crows] their row numbers, ascending
    vec* const* y_dst;         // [rows I do not own] slot row address at the owner (parity 0)
    long long parity_off_v;       // vec offset of the parity-1 slot buffer
    real* Y;                     // [n_owned_y, ldy] result
    long long ldy;
    double beta;                  // (a double for both value types, so that the host fills one struct layout)
    const long long* cptr;        // [n_crows + 1] contributions per listed row
    const int* cslot;             // slot row of each contribution, ascending source rank
    const real* slots;           // my slot buffer (parity 0)
    long long lds;
    // Atomic mode (no slots, no ordered sum): Y lives in the symmetric heap, y_dst holds the address of every
    // row I do not own inside its owner's Y, partial rows are added there with atomics.  The START phase scales
    // the owned rows that receive contributions by beta and only then signals READY; those rows (crow_flag) are
    // updated with atomics by their owner too.  Results depend on the order of the additions (not bitwise
    // reproducible).
    int atomic;
    int red_v4;                   // 1: 16-byte vector atomics also for remote rows, 0: one 4-byte atomic per value
    const unsigned char* crow_flag;  // [n_owned_y] 1: row receives contributions from peers
    PullConfig pull;              // who pulls, and in which portions
    // Pull waves, as in the SDDMM kernel: the work items are given sorted by the last wave that brings one of
    // their X rows (class 0: all columns owned); wave_items[c] = items that can run once the first c waves are
    // complete.  Long rows are cut into pieces at class boundaries (their nonzeros are sorted by class), so the
    // owned part of a hub row is computed while the pulls are in flight.
    int n_waves, tiles_per_wave;
    const int* wave_items;
    // ticket -> tile of needed X rows (null: ascending).  The host starts every rank at the peer after itself
    // on its mesh line, so that the ranks of a line read from different owners at any one time.
    const int* pull_order;
};

// Rows I own go straight into the result (Y = beta*Y + my partial; the owners' FINISH phase then adds what
// the peers pushed); rows I do not own are pushed into their slot at the owner.
struct EmitOwnedOrPush {
    vec* Yv;
    long long ldy_v;
    real beta;
    int n_owned;
    vec* const* y_dst;
    long long parity_off_v;
    __device__ __forceinline__ void operator()(int row, int v, const vec& acc) const {
        if (row < n_owned) {
            vec* y = Yv + (long long)row * ldy_v + v;
            if (beta != (real)0) { vec o = vscale(beta, *y); vadd(o, acc); *y = o; }
            else *y = acc;
        } else __stcs(ldg_ptr(y_dst + (row - n_owned)) + parity_off_v + v, acc);
    }
};

// Atomic mode of the same routing: see FusedSpmmArgs::atomic.
struct EmitOwnedOrAdd {
    vec* Yv;
    long long ldy_v;
    real beta;
    int n_owned;
    vec* const* y_dst;
    const unsigned char* crow_flag;
    int red_v4;
    __device__ __forceinline__ void operator()(int row, int v, const vec& acc) const {
        if (row < n_owned) {
            vec* y = Yv + (long long)row * ldy_v + v;
            if (__ldg(crow_flag + row)) vatomic_add(y, acc, true);  // beta was applied in the START phase
            else if (beta != (real)0) { vec o = vscale(beta, *y); vadd(o, acc); *y = o; }
            else *y = acc;
        } else {
            vec* y = ldg_ptr(y_dst + (row - n_owned)) + v;
            vatomic_add(y, acc, red_v4 != 0);
        }
    }
};

// Four resident blocks per SM (64 registers per thread) as long as a lane holds at most two vectors of a row:
// left to itself the compiler takes 128 registers for the wave bookkeeping and halves the occupancy, which costs
// the gather-bound inner loop far more than the few spills do.
// GATED: the items follow the pull waves (wave_items given).  The other form pulls everything first and carries
// no wave state: its inner loop keeps all 64 registers of a thread, which is worth 10-15 % on blocks that pull
// nothing or little (meshes 1 x Y x Z).
template <int G, int R, int U, bool ATOMIC, bool GATED>
__global__ void __launch_bounds__(256, (R <= 2 ? 4 : 2)) fused_spmm_kernel(const FusedSpmmArgs a) {
    const FusedComm& c = a.comm;
    const int lane = threadIdx.x & 31;
    const int nwarps = (int)(((long long)gridDim.x * blockDim.x) >> 5);
    const int parity = c.epoch & 1;
    extern __shared__ __align__(128) unsigned char dyn_smem[];   // bulk mode: the pullers' rings, else nothing
    __shared__ long long wave_limit[MAX_WAVES + 1];
    const bool bulk = a.pull.pullers > 0;
    const int PULL_ROWS = a.pull.tile_rows;
    BulkRing br = bulk_ring_init(dyn_smem, a.pull, threadIdx.x >> 5, lane);
    __syncthreads();
    if ((c.phases & PH_START) && !ATOMIC) start_phase(c);
    if ((c.phases & PH_START) && ATOMIC) {
        // scale the rows that peers will add to, then tell readers and contributors that this rank is ready
        if (blockIdx.x == 0 && threadIdx.x == 0) stamp(c, T_START);
        const int n_chunks = (a.n_crows + REDUCE_ROWS - 1) / REDUCE_ROWS;
        vec* Yv = reinterpret_cast<vec*>(a.Y);
        const long long ldy_v = a.ldy / VN;
        for (;;) {
            const int t = warp_ticket(c.ctrl + C_TICKET_START, lane);
            if (t >= n_chunks) break;
            const int r0 = t * REDUCE_ROWS;
            const int r1 = r0 + REDUCE_ROWS < a.n_crows ? r0 + REDUCE_ROWS : a.n_crows;
            const int total = (r1 - r0) * a.nvec;
            for (int e = lane; e < total; e += 32) {
                vec* y = Yv + (long long)__ldg(a.crows + r0 + e / a.nvec) * ldy_v + e % a.nvec;
                *y = a.beta != 0.0 ? vscale((real)a.beta, *y) : vzero((vec*)nullptr);
            }
        }
        __threadfence();
        __syncwarp();
        int old = 0;
        if (lane == 0) old = atomicAdd(c.ctrl + C_START_DONE, 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == nwarps - 1) {
            __threadfence_system();
            for (int i = lane; i < c.n_readers; i += 32) signal(c, F_READY, c.readers[i]);
            for (int i = lane; i < c.n_contrib; i += 32) signal(c, F_READY, c.contrib[i]);
        }
    }
    if (c.phases & PH_MAIN) {
        if (!(c.phases & PH_START) && blockIdx.x == 0 && threadIdx.x == 0) stamp(c, T_START);
        bool ok = wait_all(c, F_READY, c.read_from, c.n_read, W_READY);
        if (ATOMIC) ok = wait_all(c, F_READY, c.push_to, c.n_push, W_READY) && ok;
        // atomic mode, START and MAIN in one launch: my own START warps scale (or clear) the rows that receive
        // contributions with plain stores; nobody may add into them, me included, before all of them are done
        if (ATOMIC && (c.phases & PH_START)) ok = wait_counter(c, C_START_DONE, nwarps, W_READY) && ok;
        const int n_pull = (a.n_recv_x + PULL_ROWS - 1) / PULL_ROWS;
        vec* Xv = reinterpret_cast<vec*>(a.X_loc);
        const long long ldx_v = a.ldx / VN;
        const EmitOwnedOrPush emit{reinterpret_cast<vec*>(a.Y), a.ldy / VN, (real)a.beta, a.n_owned_y, a.y_dst,
                                   parity ? a.parity_off_v : 0};
        if constexpr (!GATED) {
            // pull everything (bulk mode: the puller warps; else all warps), then compute
            bool pulled = n_pull == 0;
            float4* xdst = reinterpret_cast<float4*>(Xv + (long long)a.n_owned_x * ldx_v);
            while (ok && (!bulk || (int)(threadIdx.x >> 5) < a.pull.pullers) && !aborted(c)) {
                const int t = warp_ticket(c.ctrl + C_TICKET_MAIN, lane);
                if (t >= n_pull) break;
                const int r0 = t * PULL_ROWS;
                const int r1 = r0 + PULL_ROWS < a.n_recv_x ? r0 + PULL_ROWS : a.n_recv_x;
                if (bulk) { if (!bulk_pull_tile(br, c, r0, r1, a.x_src, xdst, a.nvec, lane, true, [] {})) break; }
                else pull_rows(r0, r1, a.x_src, xdst, ldx_v, a.nvec, lane);
                __threadfence();
                __syncwarp();
                if (lane == 0 && atomicAdd(c.ctrl + C_PULLS_DONE, 1) == n_pull - 1) stamp(c, T_PULLED);
            }
            const int SPMM_ITEMS_PER_TICKET = per_ticket(a.nitems, nwarps, SPMM_ITEMS_PER_TICKET_MAX);
            while (ok) {
                const int i0 = warp_ticket(c.ctrl + C_TICKET_WORK, lane, SPMM_ITEMS_PER_TICKET);
                if (i0 >= a.nitems) break;
                if (!pulled) {
                    ok = wait_counter(c, C_PULLS_DONE, n_pull, W_PULLS);
                    pulled = true;
                    if (!ok) break;
                }
                const int i1 = i0 + SPMM_ITEMS_PER_TICKET < a.nitems ? i0 + SPMM_ITEMS_PER_TICKET : a.nitems;
                if constexpr (ATOMIC) {
                    const EmitOwnedOrAdd add{reinterpret_cast<vec*>(a.Y), a.ldy / VN, (real)a.beta, a.n_owned_y, a.y_dst,
                                             a.crow_flag, a.red_v4};
                    for (int it = i0; it < i1; ++it)
                        spmm_warp_item<real, G, R, U, EmitOwnedOrAdd, false>(__ldg(a.items + it), a.rowptr, a.colidx, a.val,
                                                                              Xv, ldx_v, a.nvec, add, a.lg, lane);
                } else {
                    for (int it = i0; it < i1; ++it)
                        spmm_warp_item<real, G, R, U, EmitOwnedOrPush, false>(__ldg(a.items + it), a.rowptr, a.colidx, a.val,
                                                                               Xv, ldx_v, a.nvec, emit, a.lg, lane);
                }
            }
        } else {
            // Pullers: in bulk mode the first warps of every block; with vector loads one warp in four, helped by any
            // warp whose own items are not ready yet.  The others start on the items that need no pulled row.
            const long long gwarp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
            const bool is_puller = bulk ? (int)(threadIdx.x >> 5) < a.pull.pullers : (gwarp & 3) == 0;
            const int n_waves = n_pull > 0 ? (a.n_waves > 0 ? a.n_waves : 1) : 0;
            // items runnable once the first w waves are complete (without wave data: none before the last pull)
            if ((int)threadIdx.x <= n_waves) {
                const int w = threadIdx.x;
                wave_limit[w] = w >= n_waves ? a.nitems : (a.wave_items ? __ldg(a.wave_items + w) : 0);
            }
            __syncthreads();
            PullGate gate;
            gate.c = c;
            gate.side[0] = {a.x_src, reinterpret_cast<float4*>(Xv + (long long)a.n_owned_x * ldx_v), a.n_recv_x};
            gate.side[1] = {nullptr, nullptr, 0};
            gate.order = a.pull_order;
            gate.limit = wave_limit;
            gate.ld_v = ldx_v;
            gate.nvec = a.nvec; gate.tile_rows = PULL_ROWS; gate.n_pull = n_pull; gate.tiles1 = 0;
            gate.tpw = a.n_waves > 0 ? a.tiles_per_wave : (n_pull > 0 ? n_pull : 1);
            gate.n_waves = n_waves;
            gate.bulk = bulk;
            gate.pulls_left = n_pull > 0 && (!bulk || is_puller);
            gate.waves_ready = 0;
        gate.pending = -1;
            gate.br = br;
            if (is_puller && ok) gate.pull_all(lane);
            const int SPMM_ITEMS_PER_TICKET = per_ticket(a.nitems, nwarps, SPMM_ITEMS_PER_TICKET_MAX);
            while (ok) {
                const int i0 = warp_ticket(c.ctrl + C_TICKET_WORK, lane, SPMM_ITEMS_PER_TICKET);
                if (i0 >= a.nitems) break;
                const int i1 = i0 + SPMM_ITEMS_PER_TICKET < a.nitems ? i0 + SPMM_ITEMS_PER_TICKET : a.nitems;
                ok = gate.ensure(i1, lane);
                if (!ok) break;
                if constexpr (ATOMIC) {
                    const EmitOwnedOrAdd add{reinterpret_cast<vec*>(a.Y), a.ldy / VN, (real)a.beta, a.n_owned_y, a.y_dst,
                                             a.crow_flag, a.red_v4};
                    for (int it = i0; it < i1; ++it)
                        spmm_warp_item<real, G, R, U, EmitOwnedOrAdd, false>(__ldg(a.items + it), a.rowptr, a.colidx, a.val,
                                                                              Xv, ldx_v, a.nvec, add, a.lg, lane);
                } else {
                    for (int it = i0; it < i1; ++it)
                        spmm_warp_item<real, G, R, U, EmitOwnedOrPush, false>(__ldg(a.items + it), a.rowptr, a.colidx, a.val,
                                                                               Xv, ldx_v, a.nvec, emit, a.lg, lane);
                }
            }
            if (ok) gate.pull_all(lane);  // no item left but tiles remain (tiny blocks)
        }
        main_epilogue(c, lane, nwarps);
    }
    if (c.phases & PH_FINISH) {
        bool ok = wait_all(c, F_PART, c.contrib, c.n_contrib, W_PART);
        // my own partial rows come from my own MAIN warps (same launch): wait for all of them
        if (ok && (c.phases & PH_MAIN)) ok = wait_counter(c, C_MAIN_DONE, nwarps, W_PART);
        // only rows that receive contributions are touched: crows lists them, cptr/cslot their slot rows in
        // ascending source order
        const int n_chunks = (a.n_crows + REDUCE_ROWS - 1) / REDUCE_ROWS;
        const vec* Sv = reinterpret_cast<const vec*>(a.slots) + (parity ? a.parity_off_v : 0);
        vec* Yv = reinterpret_cast<vec*>(a.Y);
        const long long lds_v = a.lds / VN, ldy_v = a.ldy / VN;
        while (ok && !ATOMIC) {  // atomic mode: the contributions are already in Y
            const int t = warp_ticket(c.ctrl + C_TICKET_FIN, lane);
            if (t >= n_chunks) break;
            const int r0 = t * REDUCE_ROWS;
            const int r1 = r0 + REDUCE_ROWS < a.n_crows ? r0 + REDUCE_ROWS : a.n_crows;
            const int total = (r1 - r0) * a.nvec;
            // two elements per lane and step: their loads (own row, slot rows) are independent and overlap
            for (int e = lane; e < total; e += 64) {
                vec s[2];
                vec* y[2];
                long long p0[2], p1[2];
                int vv[2];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int eq = e + 32 * q;
                    y[q] = nullptr;
                    if (eq < total) {
                        const int ci = r0 + eq / a.nvec;
                        vv[q] = eq % a.nvec;
                        y[q] = Yv + (long long)__ldg(a.crows + ci) * ldy_v + vv[q];
                        p0[q] = __ldg(a.cptr + ci);
                        p1[q] = __ldg(a.cptr + ci + 1);
                    }
                }
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    if (y[q]) s[q] = *y[q];
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    if (y[q])
                        for (long long p = p0[q]; p < p1[q]; ++p)
                            vadd(s[q], __ldcg(Sv + (long long)__ldg(a.cslot + p) * lds_v + vv[q]));
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    if (y[q]) *y[q] = s[q];
            }
        }
        finish_epilogue(c, lane, nwarps);
    }
}

}  // namespace SP3_FUSED_NS
}  // namespace sp3

using namespace sp3;
using namespace sp3::SP3_FUSED_NS;

// Arguments arrive as a packed struct prepared by the Python front end (see
// spcomm3d_b200/ops/fused.py for the field order); `args` points to host memory.
#if SP3_FUSED_IS_F32
SP3_API int sp3_fused_struct_sizes(int* sddmm_bytes, int* spmm_bytes, int* comm_bytes) {
    *sddmm_bytes = (int)sizeof(FusedSddmmArgs);
    *spmm_bytes = (int)sizeof(FusedSpmmArgs);
    *comm_bytes = (int)sizeof(FusedComm);
    return 0;
}
#endif

// The kernels synchronise their own warps through grid-wide counters, so every block of the grid has to be
// resident at once.  A cooperative launch gives that guarantee: the grid is sized from the occupancy query and
// the launch fails with an error (instead of a kernel that waits for blocks that never start) if the device
// cannot hold it.
template <typename K, typename A>
static int launch_resident(K kernel, const A& args, cudaStream_t st) {
    A copy = args;
    void* params[] = {&copy};
    if (args.pull.pullers < 0 || args.pull.pullers > BULK_MAX_PULLERS || args.pull.tile_rows < 1 ||
        (args.pull.pullers > 0 && (args.pull.stage_bytes < 1024 || args.pull.stage_bytes % 16)))
        return (int)cudaErrorInvalidValue;
    const size_t smem = bulk_smem_bytes(args.pull);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const unsigned blocks = persistent_blocks(kernel, 0, 256, smem);
    return (int)cudaLaunchCooperativeKernel((const void*)kernel, dim3(blocks), dim3(256), params, smem, st);
}

#define SP3_FUSED_CAT2(a, b) a##b
#define SP3_FUSED_CAT(a, b) SP3_FUSED_CAT2(a, b)

SP3_API int SP3_FUSED_CAT(sp3_fused_sddmm_, SP3_FUSED_SUFFIX)(const void* args, void* stream) {
    FusedSddmmArgs a = *reinterpret_cast<const FusedSddmmArgs*>(args);
    cudaStream_t st = (cudaStream_t)stream;
    if (a.n_waves > MAX_WAVES) return (int)cudaErrorInvalidValue;
#if !SP3_FUSED_IS_F32
    if (a.direct_push == 3) return (int)cudaErrorInvalidValue;   // the in-switch reduction is built for fp32 only
#endif
    cudaError_t e = cudaMemsetAsync(a.comm.ctrl, 0, C_WORDS * sizeof(int), st);
    if (e != cudaSuccess) return (int)e;
    int G, R, rc = 0;
    pick_shape(a.nvec, &G, &R, false);
#define SP3_FSDDMM(GG, RR) rc = launch_resident(fused_sddmm_kernel<GG, RR, (RR >= 8 ? 2 : 4)>, a, st)
    SP3_DISPATCH_GR(SP3_FSDDMM)
#undef SP3_FSDDMM
    return rc ? rc : (int)cudaGetLastError();
}

SP3_API int SP3_FUSED_CAT(sp3_fused_spmm_, SP3_FUSED_SUFFIX)(const void* args, void* stream) {
    FusedSpmmArgs a = *reinterpret_cast<const FusedSpmmArgs*>(args);
    cudaStream_t st = (cudaStream_t)stream;
    if (a.n_waves > MAX_WAVES) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaMemsetAsync(a.comm.ctrl, 0, C_WORDS * sizeof(int), st);
    if (e != cudaSuccess) return (int)e;
    int G, R, rc = 0;
    pick_shape(a.nvec, &G, &R, true);
    const bool gated = a.wave_items != nullptr && a.n_waves > 0 && a.n_recv_x > 0;
#define SP3_FSPMM(GG, RR)                                                                        \
    rc = a.atomic ? (gated ? launch_resident(fused_spmm_kernel<GG, RR, (RR >= 8 ? 2 : 4), true, true>, a, st)     \
                           : launch_resident(fused_spmm_kernel<GG, RR, (RR >= 8 ? 2 : 4), true, false>, a, st))   \
                  : (gated ? launch_resident(fused_spmm_kernel<GG, RR, (RR >= 8 ? 2 : 4), false, true>, a, st)    \
                           : launch_resident(fused_spmm_kernel<GG, RR, (RR >= 8 ? 2 : 4), false, false>, a, st))
    SP3_DISPATCH_GR(SP3_FSPMM)
#undef SP3_FSPMM
    return rc ? rc : (int)cudaGetLastError();
}

#if SP3_FUSED_IS_F32
// Number of int32 words the caller must provide as `ctrl`.
SP3_API int sp3_fused_ctrl_words() { return C_WORDS; }
#endif

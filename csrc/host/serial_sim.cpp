// Analytic communication-volume simulator for any X x Y processor mesh, and
// the memory-excess metric of the sparsity-agnostic method.  No communication
// library is involved: everything is counted from the sparsity pattern.
//
// Counterparts in the reference: miniapp/serialSim.cpp:109-252 (exact sparse
// send/receive messages and rows per processor, closed-form dense volumes)
// and miniapp/countExcess.cpp:135-155.  Unlike the mask-based planner this
// code has no limit on the mesh line length (the reference sweeps P up to
// 32768): touch sets are built by sorting (id, coordinate) pairs.
#include "sp3_host.hpp"

#include <algorithm>
#include <cstring>
#include <numeric>
#include <vector>

extern "C" int sp3_rr_map(uint64_t n, uint32_t parts, uint64_t seed, uint64_t stream, int32_t* map);

namespace {

struct SideResult {
    std::vector<uint64_t> send_vol, recv_vol, send_msg, recv_msg;  // per xy rank
    std::vector<uint64_t> owned, touched;                          // per xy rank
    std::vector<uint64_t> line_size;                               // ids per mesh line
};

// One side (row side: ids = rows, line = rowmap, free axis = y of colmap).
// rank_of(line, free) gives the xy rank.
template <typename RankOf>
SideResult simulate_side(uint64_t nnz, const uint32_t* ids, const uint32_t* others, uint64_t n,
                         const int32_t* linemap, uint32_t nlines, const int32_t* freemap, uint32_t nfree,
                         int policy, uint64_t seed, uint64_t stream, uint32_t P, RankOf rank_of) {
    SideResult res;
    res.send_vol.assign(P, 0); res.recv_vol.assign(P, 0); res.send_msg.assign(P, 0); res.recv_msg.assign(P, 0);
    res.owned.assign(P, 0); res.touched.assign(P, 0); res.line_size.assign(nlines, 0);
    // distinct (id, free coordinate) pairs
    std::vector<uint64_t> keys(nnz);
    for (uint64_t i = 0; i < nnz; ++i) keys[i] = (uint64_t)ids[i] * nfree + (uint32_t)freemap[others[i]];
    std::sort(keys.begin(), keys.end());
    keys.erase(std::unique(keys.begin(), keys.end()), keys.end());
    std::vector<uint64_t> start(n + 1, 0);
    for (uint64_t k : keys) ++start[k / nfree + 1];
    for (uint64_t i = 0; i < n; ++i) start[i + 1] += start[i];
    // pair_seen[line][owner][receiver] for message counting
    std::vector<uint8_t> seen((size_t)nlines * nfree * nfree, 0);
    std::vector<uint64_t> rr(nlines, 0);
    for (uint64_t id = 0; id < n; ++id) {
        const uint32_t line = (uint32_t)linemap[id];
        ++res.line_size[line];
        const uint64_t b = start[id], e = start[id + 1];
        uint32_t owner;
        if (e == b || policy == 1) owner = (uint32_t)(rr[line]++ % nfree);
        else owner = (uint32_t)(keys[b + sp3::rnd(seed, stream, id) % (e - b)] % nfree);
        const uint32_t orank = rank_of(line, owner);
        ++res.owned[orank];
        for (uint64_t t = b; t < e; ++t) {
            const uint32_t f = (uint32_t)(keys[t] % nfree);
            ++res.touched[rank_of(line, f)];
            if (f == owner) continue;
            ++res.recv_vol[rank_of(line, f)];
            ++res.send_vol[orank];
            uint8_t& s = seen[((size_t)line * nfree + owner) * nfree + f];
            if (!s) { s = 1; ++res.send_msg[orank]; ++res.recv_msg[rank_of(line, f)]; }
        }
    }
    return res;
}

void summarize(const std::vector<uint64_t>& v, double* avg, double* mx) {
    uint64_t s = 0, m = 0;
    for (auto x : v) { s += x; m = std::max(m, x); }
    *avg = v.empty() ? 0.0 : (double)s / (double)v.size();
    *mx = (double)m;
}

}  // namespace

// mode 0 = SDDMM pre-communication (A rows + B rows), 1 = SpMM pre (X rows
// only), 2 = SpMM post (partial Y rows to owners: the row side reversed).
// out[0..7]  sparse: avgSendMsgs avgSendVol avgRecvMsgs avgRecvVol maxSendMsgs maxSendVol maxRecvMsgs maxRecvVol
// out[8..15] dense (whole-slab broadcast), same order.  Volumes are in dense
// rows; multiply by k/Z for elements.
SP3_API int sp3_serial_sim(uint64_t nnz, const uint32_t* rows, const uint32_t* cols, uint64_t M, uint64_t N,
                           uint32_t X, uint32_t Y, uint64_t seed, int policy, int mode, double* out) {
    if (X == 0 || Y == 0) return sp3::E_ARG;
    // mode + 16: the dense method is counted as the reference's simulator counts it (serialSim.cpp:233-247):
    // one message to, and one copy of the own block for, every other rank of the line
    const bool p2p_dense = (mode & 16) != 0;
    mode &= 15;
    const uint32_t P = X * Y;
    std::vector<int32_t> rowmap(M), colmap(N);
    sp3_rr_map(M, X, seed, 101, rowmap.data());
    sp3_rr_map(N, Y, seed, 102, colmap.data());
    auto row_rank = [Y](uint32_t x, uint32_t y) { return x * Y + y; };
    auto col_rank = [Y](uint32_t y, uint32_t x) { return x * Y + y; };
    SideResult R = simulate_side(nnz, rows, cols, M, rowmap.data(), X, colmap.data(), Y, policy, seed, 103, P, row_rank);
    SideResult Cc = simulate_side(nnz, cols, rows, N, colmap.data(), Y, rowmap.data(), X, policy, seed, 104, P, col_rank);
    std::vector<uint64_t> sv(P), rv(P), sm(P), rm(P), dsv(P), drv(P), dsm(P), drm(P);
    for (uint32_t p = 0; p < P; ++p) {
        const uint32_t x = p / Y, y = p % Y;
        const bool useR = mode != 1, useC = mode != 2;
        if (mode == 2) {  // roles swapped: partial rows flow to owners
            sv[p] = R.recv_vol[p]; rv[p] = R.send_vol[p]; sm[p] = R.recv_msg[p]; rm[p] = R.send_msg[p];
        } else {
            sv[p] = (useR ? R.send_vol[p] : 0) + (useC ? Cc.send_vol[p] : 0);
            rv[p] = (useR ? R.recv_vol[p] : 0) + (useC ? Cc.recv_vol[p] : 0);
            sm[p] = (useR ? R.send_msg[p] : 0) + (useC ? Cc.send_msg[p] : 0);
            rm[p] = (useR ? R.recv_msg[p] : 0) + (useC ? Cc.recv_msg[p] : 0);
        }
        // dense: broadcast own block once per side, receive every other block of the line
        dsv[p] = (useR ? R.owned[p] : 0) + (useC ? Cc.owned[p] : 0);
        drv[p] = (useR ? R.line_size[x] - R.owned[p] : 0) + (useC ? Cc.line_size[y] - Cc.owned[p] : 0);
        dsm[p] = (useR ? 1 : 0) + (useC ? 1 : 0);
        drm[p] = (useR ? Y - 1 : 0) + (useC ? X - 1 : 0);
        if (p2p_dense) {
            dsv[p] = (useR ? R.owned[p] * (Y - 1) : 0) + (useC ? Cc.owned[p] * (X - 1) : 0);
            dsm[p] = drm[p];
        }
    }
    summarize(sm, &out[0], &out[4]); summarize(sv, &out[1], &out[5]);
    summarize(rm, &out[2], &out[6]); summarize(rv, &out[3], &out[7]);
    summarize(dsm, &out[8], &out[12]); summarize(dsv, &out[9], &out[13]);
    summarize(drm, &out[10], &out[14]); summarize(drv, &out[11], &out[15]);
    return sp3::OK;
}

// out[0] = sum over ranks of dense rows the sparsity-agnostic method stores
// (whole A slab of the mesh row + whole B slab of the mesh column), out[1] =
// sum over ranks of dense rows actually touched by the rank's block, out[2] =
// excess = out[0] - out[1].
SP3_API int sp3_count_excess(uint64_t nnz, const uint32_t* rows, const uint32_t* cols, uint64_t M, uint64_t N,
                             uint32_t X, uint32_t Y, uint64_t seed, double* out) {
    if (X == 0 || Y == 0) return sp3::E_ARG;
    const uint32_t P = X * Y;
    std::vector<int32_t> rowmap(M), colmap(N);
    sp3_rr_map(M, X, seed, 101, rowmap.data());
    sp3_rr_map(N, Y, seed, 102, colmap.data());
    auto row_rank = [Y](uint32_t x, uint32_t y) { return x * Y + y; };
    auto col_rank = [Y](uint32_t y, uint32_t x) { return x * Y + y; };
    SideResult R = simulate_side(nnz, rows, cols, M, rowmap.data(), X, colmap.data(), Y, 0, seed, 103, P, row_rank);
    SideResult Cc = simulate_side(nnz, cols, rows, N, colmap.data(), Y, rowmap.data(), X, 0, seed, 104, P, col_rank);
    double stored = 0, touched = 0;
    for (uint32_t p = 0; p < P; ++p) {
        stored += (double)R.line_size[p / Y] + (double)Cc.line_size[p % Y];
        touched += (double)R.touched[p] + (double)Cc.touched[p];
    }
    out[0] = stored; out[1] = touched; out[2] = stored - touched;
    return sp3::OK;
}

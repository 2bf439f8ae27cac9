// Timing driver for the reference library (nfabubaker/SpComm3D).
//
//   ref_driver -k K -c Z -s STEPS -w WARMUP [-t SECONDS] matrix.bin
//
// Links the reference's own, unmodified sources (src/*.cpp, src/*.hpp) and
// calls its public functions in the order its benchmarks do
// (miniapp/bench_both.cpp:122-236, miniapp/bench_spmm.cpp:122-188): collective
// read + 2D distribution, index localisation, ownership, plan setup, and then
// the distributed kernels -- SDDMM "sparse" (dist_sddmm_spcomm), SDDMM
// "sparseNB" (dist_sddmm_spcomm3) and SpMM "sparse" (dist_spmm_spcomm).  The
// only things added are the warm-up/step counts and a nanosecond clock around
// each call (the reference's own timers are integer milliseconds); each step
// is preceded by a barrier and its time is the maximum over ranks.  -t gives
// every kernel a wall-clock allowance: warm-up stops after a quarter of it and
// the timed steps after all of it (at least one of each runs); the counts that
// were actually run are printed.
// Rank 0 prints one line starting with REFDRIVER followed by JSON.
#include <algorithm>
#include <array>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "mpi.h"
#include "basic.hpp"
#include "SparseMatrix.hpp"
#include "comm.hpp"
#include "denseComm.hpp"
#include "parallel_io.hpp"
#include "distribute.hpp"
#include "comm_setup.hpp"
#include "distributed_comp.hpp"

using namespace SpKernels;
using namespace DComm;
using clk = std::chrono::steady_clock;

static double max_ms(double local_ms, MPI_Comm comm) {
    double out = 0;
    MPI_Allreduce(&local_ms, &out, 1, MPI_DOUBLE, MPI_MAX, comm);
    return out;
}

struct Timed { double ms; int steps, warmup; };

template <typename F> static Timed time_steps(F&& step, int warmup, int steps, double budget_s, MPI_Comm comm) {
    // every rank takes the same decisions: the elapsed time they compare is the maximum over ranks
    const auto begin = clk::now();
    auto elapsed_s = [&] { return max_ms(std::chrono::duration<double, std::milli>(clk::now() - begin).count(), comm) / 1e3; };
    int w = 0, n = 0;
    for (; w < warmup; ++w) {
        if (w > 0 && budget_s > 0 && elapsed_s() > budget_s / 4) break;
        step();
    }
    double total = 0;
    for (; n < steps; ++n) {
        if (n > 0 && budget_s > 0 && elapsed_s() > budget_s) break;
        MPI_Barrier(comm);
        auto t0 = clk::now();
        step();
        double ms = std::chrono::duration<double, std::milli>(clk::now() - t0).count();
        total += max_ms(ms, comm);
    }
    return {total / std::max(1, n), n, w};
}

int main(int argc, char** argv) {
    MPI_Init(&argc, &argv);
    int rank, size;
    MPI_Comm comm = MPI_COMM_WORLD, xycomm, zcomm, cartcomm;
    MPI_Comm_rank(comm, &rank);
    MPI_Comm_size(comm, &size);
    idx_t f = 32; int c = 1, steps = 3, warmup = 1; double budget_s = 0; std::string filename;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "-k") && i + 1 < argc) f = (idx_t)atoi(argv[++i]);
        else if (!strcmp(argv[i], "-c") && i + 1 < argc) c = atoi(argv[++i]);
        else if (!strcmp(argv[i], "-s") && i + 1 < argc) steps = atoi(argv[++i]);
        else if (!strcmp(argv[i], "-w") && i + 1 < argc) warmup = atoi(argv[++i]);
        else if (!strcmp(argv[i], "-t") && i + 1 < argc) budget_s = atof(argv[++i]);
        else filename = argv[i];
    }
    if (filename.empty()) { if (!rank) fprintf(stderr, "usage: ref_driver -k K -c Z -s STEPS -w WARMUP [-t SECONDS] matrix.bin\n"); MPI_Finalize(); return 2; }
    std::string mtxName = filename.substr(filename.find_last_of("/\\") + 1);
    mtxName = mtxName.substr(0, mtxName.find_last_of('.'));

    std::array<int, 3> dims = {0, 0, c}, zeroArr = {0, 0, 0};
    MPI_Dims_create(size, 3, dims.data());
    MPI_Cart_create(comm, 3, dims.data(), zeroArr.data(), 0, &cartcomm);
    const int Z = dims[2];
    std::array<int, 3> remain = {true, true, false};
    MPI_Cart_sub(cartcomm, remain.data(), &xycomm);
    remain = {false, false, true};
    MPI_Cart_sub(cartcomm, remain.data(), &zcomm);
    int myxyrank, myz;
    MPI_Comm_rank(xycomm, &myxyrank);
    MPI_Comm_rank(zcomm, &myz);

    auto s0 = clk::now();
    cooMat Cloc, Sloc;
    Sloc.mtxName = mtxName;
    std::vector<int> rpvec, cpvec;
    {
        std::vector<int> rpvec2D, cpvec2D;
        read_bin_parallel_distribute_coo(filename, Sloc, rpvec2D, cpvec2D, cartcomm, xycomm, zcomm);
        Sloc.localizeIndices();
        Cloc = Sloc;
        Cloc.rank = rank; Sloc.rank = rank;
        Cloc.zrank = myz; Sloc.zrank = myz;
        distribute3D_AB_respect_communication(rpvec2D, cpvec2D, rpvec, cpvec, Cloc, xycomm, zcomm, cartcomm);
    }
    const double setup_ms = max_ms(std::chrono::duration<double, std::milli>(clk::now() - s0).count(), comm);
    idx_t floc = f / Z;
    if (f % Z > 0 && (idx_t)myz < f % Z) ++floc;

    Timed sddmm_sparse, sddmm_nb, spmm;
    {   // SDDMM, combined expand handle with send and receive staging
        for (auto& e : Cloc.vv) e = 0.0;
        SparseComm<real_t> comm_expand; DenseComm comm_reduce;
        denseMatrix Aloc, Bloc;
        Aloc.m = Cloc.nrows; Aloc.n = floc; Bloc.m = Cloc.ncols; Bloc.n = floc;
        Aloc.data.resize((size_t)Aloc.m * Aloc.n, myxyrank + 1);
        Bloc.data.resize((size_t)Bloc.m * Bloc.n, myxyrank + 1);
        setup_3dsddmm(Cloc, f, c, xycomm, zcomm, Aloc, Bloc, rpvec, cpvec, comm_expand, comm_reduce);
        sddmm_sparse = time_steps([&] { dist_sddmm_spcomm(Aloc, Bloc, Sloc, comm_expand, comm_reduce, Cloc, cartcomm); },
                                     warmup, steps, budget_s, comm);
    }
    {   // SDDMM, zero staging (derived datatypes, receive in place)
        for (auto& e : Cloc.vv) e = 0.0;
        std::fill(Cloc.ownedVals.begin(), Cloc.ownedVals.end(), 0.0);
        SparseComm<real_t> eA, eB; DenseComm comm_reduce;
        denseMatrix Aloc, Bloc;
        Aloc.m = Cloc.nrows; Aloc.n = floc; Bloc.m = Cloc.ncols; Bloc.n = floc;
        Aloc.data.resize((size_t)Aloc.m * Aloc.n, myxyrank + 1);
        Bloc.data.resize((size_t)Bloc.m * Bloc.n, myxyrank + 1);
        std::vector<idx_t> mapA(Aloc.m, -1), mapB(Bloc.m, -1), mapAI(Aloc.m), mapBI(Bloc.m);
        setup_3dsddmm_NoBuffers(Cloc, f, c, xycomm, zcomm, Aloc, Bloc, rpvec, cpvec, eA, eB, comm_reduce, mapA, mapB);
        for (idx_t i = 0; i < Aloc.m; ++i) mapAI[mapA[i]] = i;
        for (idx_t i = 0; i < Bloc.m; ++i) mapBI[mapB[i]] = i;
        Sloc.ReMapIndices(mapA, mapB);
        Cloc.ReMapIndices(mapA, mapB);
        sddmm_nb = time_steps([&] { dist_sddmm_spcomm3(Aloc, Bloc, Sloc, eA, eB, comm_reduce, Cloc, cartcomm); },
                                 warmup, steps, budget_s, comm);
        Sloc.ReMapIndices(mapAI, mapBI);
        Cloc.ReMapIndices(mapAI, mapBI);
    }
    {   // SpMM
        SparseComm<real_t> comm_expand, comm_reduce;
        denseMatrix Yloc, Xloc;
        Yloc.m = Sloc.nrows; Yloc.n = floc; Xloc.m = Sloc.ncols; Xloc.n = floc;
        Yloc.data.resize((size_t)Yloc.m * Yloc.n, myxyrank + 1);
        Xloc.data.resize((size_t)Xloc.m * Xloc.n, myxyrank + 1);
        setup_spmm(Sloc, f, c, xycomm, zcomm, Xloc, Yloc, rpvec, cpvec, comm_expand, comm_reduce);
        spmm = time_steps([&] { dist_spmm_spcomm(Xloc, Sloc, Yloc, comm_expand, comm_reduce, cartcomm); },
                             warmup, steps, budget_s, comm);
    }
    fflush(stdout);
    MPI_Barrier(comm);
    if (rank == 0) {
        const int steps_run = std::min(sddmm_sparse.steps, std::min(sddmm_nb.steps, spmm.steps));
        const int warmup_run = std::min(sddmm_sparse.warmup, std::min(sddmm_nb.warmup, spmm.warmup));
        printf("REFDRIVER {\"ranks\": %d, \"mesh\": \"%dx%dx%d\", \"k\": %u, \"gnnz\": %lu, \"steps\": %d, \"warmup\": %d, "
               "\"steps_by_kernel\": [%d, %d, %d], \"budget_s\": %.1f, "
               "\"sddmm_sparse_ms\": %.6f, \"sddmm_sparseNB_ms\": %.6f, \"spmm_sparse_ms\": %.6f, \"setup_ms\": %.3f}\n",
               size, dims[0], dims[1], dims[2], f, (unsigned long)Sloc.gnnz, steps_run, warmup_run,
               sddmm_sparse.steps, sddmm_nb.steps, spmm.steps, budget_s,
               sddmm_sparse.ms, sddmm_nb.ms, spmm.ms, setup_ms);
        fflush(stdout);
    }
    MPI_Comm_free(&xycomm);
    MPI_Comm_free(&zcomm);
    MPI_Comm_free(&cartcomm);
    MPI_Finalize();
    return 0;
}

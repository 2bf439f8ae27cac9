// Calls the reference's SpMM loop (src/core_ops.cpp:24-35) on a MatrixMarket
// file read by the reference's own reader (src/mm.hpp) and prints the sum and
// the sum of squares of Y.  X[i][j] = (i % 97) / 100 + j / 1000, Y starts at
// zero.  The reference has no SpMM checker of its own; this gives the tests a
// second opinion from its code.  Usage: ref_spmm_check <k> <file.mtx>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "basic.hpp"
#include "mm.hpp"
#include "SparseMatrix.hpp"
#include "core_ops.hpp"

using namespace SpKernels;

int main(int argc, char** argv) {
    if (argc != 3) { std::fprintf(stderr, "usage: %s <k> <file.mtx>\n", argv[0]); return 2; }
    const idx_t k = (idx_t)std::atoi(argv[1]);
    std::string fn = argv[2];
    cooMat S;
    mm reader(fn);
    reader.read_mm(fn, S);
    denseMatrix X, Y;
    X.m = S.gncols; X.n = k;
    Y.m = S.gnrows; Y.n = k;
    X.data.resize((size_t)X.m * X.n);
    Y.data.assign((size_t)Y.m * Y.n, 0.0);
    for (size_t i = 0; i < X.m; ++i)
        for (size_t j = 0; j < X.n; ++j) X.at(i, j) = (real_t)(i % 97) / 100 + (real_t)j / 1000;
    spmm(X, S, Y);
    long double s = 0, s2 = 0;
    for (double v : Y.data) { s += v; s2 += (long double)v * v; }
    std::printf("%.12Lg %.12Lg\n", s, s2);
    return 0;
}

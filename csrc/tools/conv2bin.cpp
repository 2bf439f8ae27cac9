// conv2bin: MatrixMarket (.mtx) -> binary (.bin) converter, standalone.
//
//   conv2bin [-o out.bin] [-d] in.mtx
//
// Output: u32 nrows, u32 ncols, u64 nnz, then nnz x {u32 row, u32 col, f64
// val}; byte-identical to the reference tool tools/read_convert_mm.cpp:81-94
// (default output name = input with the extension replaced by .bin, :124-126).
// -d stores the diagonal of a symmetric matrix once instead of mirroring it
// (the reference always mirrors, src/mm.hpp:53-57).  -z is accepted and
// ignored, as in the reference (:55-57).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

extern "C" {
int sp3_mm_read_header(const char*, uint64_t*, uint64_t*, uint64_t*, uint64_t*, int*);
int sp3_mm_read(const char*, uint64_t, int, uint32_t*, uint32_t*, double*, uint64_t*);
int sp3_bin_write(const char*, uint32_t, uint32_t, uint64_t, const uint32_t*, const uint32_t*, const double*,
                  const float*);
}

static void usage(const char* prog) {
    fprintf(stderr, "usage: %s [-o out.bin] [-d] [-z Z] in.mtx\n", prog);
}

int main(int argc, char** argv) {
    std::string in, out;
    int mirror_diag = 1;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "-o") && i + 1 < argc) out = argv[++i];
        else if (!strcmp(argv[i], "-z") && i + 1 < argc) ++i;
        else if (!strcmp(argv[i], "-d")) mirror_diag = 0;
        else if (!strcmp(argv[i], "-h")) { usage(argv[0]); return 0; }
        else if (argv[i][0] == '-') { usage(argv[0]); return 2; }
        else in = argv[i];
    }
    if (in.empty()) { usage(argv[0]); return 2; }
    if (out.empty()) {
        size_t dot = in.find_last_of('.');
        out = (dot == std::string::npos ? in : in.substr(0, dot)) + ".bin";
    }
    uint64_t nr, nc, fnnz, cap, nnz = 0;
    int flags;
    int rc = sp3_mm_read_header(in.c_str(), &nr, &nc, &fnnz, &cap, &flags);
    if (rc) { fprintf(stderr, "conv2bin: cannot read header of %s (error %d)\n", in.c_str(), rc); return 1; }
    std::vector<uint32_t> rows(cap), cols(cap);
    std::vector<double> vals(cap);
    rc = sp3_mm_read(in.c_str(), cap, mirror_diag, rows.data(), cols.data(), vals.data(), &nnz);
    if (rc) { fprintf(stderr, "conv2bin: cannot parse %s (error %d)\n", in.c_str(), rc); return 1; }
    rc = sp3_bin_write(out.c_str(), (uint32_t)nr, (uint32_t)nc, nnz, rows.data(), cols.data(), vals.data(), nullptr);
    if (rc) { fprintf(stderr, "conv2bin: cannot write %s (error %d)\n", out.c_str(), rc); return 1; }
    printf("%s: %lu x %lu, %lu nonzeros -> %s\n", in.c_str(), nr, nc, nnz, out.c_str());
    return 0;
}

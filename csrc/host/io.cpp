// Matrix file I/O: the conv2bin binary format and the MatrixMarket reader.
//
// Binary layout (little endian), byte-compatible with the reference writer
// tools/read_convert_mm.cpp:81-94 and its reader src/parallel_io.hpp:59-63:
//   u32 nrows, u32 ncols, u64 nnz, then nnz x { u32 row, u32 col, f64 val }.
// Rows/cols are 0-based, entries keep the order of the source file.
//
// Unlike the reference (one MPI_File_read per nonzero, parallel_io.hpp:93-94)
// a rank reads its whole [start, start+count) slice with one pread loop.
#include "sp3_host.hpp"

#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/stat.h>
#include <unistd.h>
#include <new>
#include <vector>

namespace {
#pragma pack(push, 1)
struct BinHeader { uint32_t nrows, ncols; uint64_t nnz; };
struct BinTriplet { uint32_t row, col; double val; };
#pragma pack(pop)
static_assert(sizeof(BinHeader) == 16, "header is 16 bytes");
static_assert(sizeof(BinTriplet) == 16, "triplet is 16 bytes");

int pread_all(int fd, void* buf, size_t bytes, off_t off) {
    char* p = (char*)buf;
    while (bytes) {
        ssize_t got = pread(fd, p, bytes, off);
        if (got < 0) { if (errno == EINTR) continue; return sp3::E_IO; }
        if (got == 0) return sp3::E_FORMAT;  // truncated file
        p += got; off += got; bytes -= (size_t)got;
    }
    return sp3::OK;
}
}  // namespace

SP3_API int sp3_bin_read_header(const char* path, uint32_t* nrows, uint32_t* ncols, uint64_t* nnz) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return sp3::E_IO;
    BinHeader h;
    int rc = pread_all(fd, &h, sizeof h, 0);
    struct stat st;
    if (rc == sp3::OK && fstat(fd, &st) == 0) {
        // divide instead of multiplying: a corrupt count near 2^64 must not wrap past the check
        if ((uint64_t)st.st_size < sizeof(BinHeader) ||
            h.nnz > ((uint64_t)st.st_size - sizeof(BinHeader)) / sizeof(BinTriplet)) rc = sp3::E_FORMAT;
    }
    close(fd);
    if (rc != sp3::OK) return rc;
    *nrows = h.nrows; *ncols = h.ncols; *nnz = h.nnz;
    return sp3::OK;
}

// Reads triplets [start, start+count) into split arrays.  `vals32` or
// `vals64` may be null; whichever is non-null receives the values.
SP3_API int sp3_bin_read_range(const char* path, uint64_t start, uint64_t count,
                               uint32_t* rows, uint32_t* cols, double* vals64, float* vals32) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return sp3::E_IO;
    BinHeader h;
    int rc = pread_all(fd, &h, sizeof h, 0);
    if (rc == sp3::OK && (start > h.nnz || count > h.nnz - start)) rc = sp3::E_RANGE;
    const size_t CH = 1u << 20;
    std::vector<BinTriplet> buf;
    if (rc == sp3::OK) {
        try { buf.resize(count < CH ? (size_t)count : CH); }
        catch (const std::bad_alloc&) { rc = sp3::E_IO; }  // nothing may be thrown across the C interface
    }
    for (uint64_t done = 0; rc == sp3::OK && done < count;) {
        size_t n = (size_t)((count - done) < CH ? (count - done) : CH);
        rc = pread_all(fd, buf.data(), n * sizeof(BinTriplet),
                       (off_t)(sizeof(BinHeader) + (start + done) * sizeof(BinTriplet)));
        if (rc != sp3::OK) break;
        for (size_t i = 0; i < n; ++i) {
            if (buf[i].row >= h.nrows || buf[i].col >= h.ncols) { rc = sp3::E_RANGE; break; }
            rows[done + i] = buf[i].row;
            cols[done + i] = buf[i].col;
            if (vals64) vals64[done + i] = buf[i].val;
            if (vals32) vals32[done + i] = (float)buf[i].val;
        }
        done += n;
    }
    close(fd);
    return rc;
}

SP3_API int sp3_bin_write(const char* path, uint32_t nrows, uint32_t ncols, uint64_t nnz,
                          const uint32_t* rows, const uint32_t* cols,
                          const double* vals64, const float* vals32) {
    FILE* f = fopen(path, "wb");
    if (!f) return sp3::E_IO;
    BinHeader h{nrows, ncols, nnz};
    int rc = fwrite(&h, sizeof h, 1, f) == 1 ? sp3::OK : sp3::E_IO;
    const size_t CH = 1u << 20;
    std::vector<BinTriplet> buf(nnz < CH ? (size_t)nnz : CH);
    for (uint64_t done = 0; rc == sp3::OK && done < nnz;) {
        size_t n = (size_t)((nnz - done) < CH ? (nnz - done) : CH);
        for (size_t i = 0; i < n; ++i) {
            buf[i].row = rows[done + i];
            buf[i].col = cols[done + i];
            buf[i].val = vals64 ? vals64[done + i] : (vals32 ? (double)vals32[done + i] : 1.0);
        }
        if (fwrite(buf.data(), sizeof(BinTriplet), n, f) != n) rc = sp3::E_IO;
        done += n;
    }
    if (fclose(f) != 0 && rc == sp3::OK) rc = sp3::E_IO;
    return rc;
}

// ---------------------------------------------------------------------------
// MatrixMarket coordinate reader.  Semantics follow the reference parser
// src/mm.hpp:20-74: the banner is searched for "pattern", "symmetric" and
// "complex"; '%' comment lines are skipped; indices become 0-based; pattern
// entries get value 1.0; the imaginary part of complex entries is dropped.
// Symmetric files are expanded.  With mirror_diagonal != 0 every entry is
// mirrored, diagonals included, into the second half of the arrays (what the
// reference does, mm.hpp:32,53-57, so .bin output is byte-identical); with 0
// diagonal entries are stored once and the returned nnz is smaller.
// ---------------------------------------------------------------------------
namespace {
struct MMInfo { uint64_t nrows, ncols, file_nnz; bool pattern, symm, cplx; long data_off; };

int mm_parse_header(FILE* f, MMInfo* info) {
    char line[4096];
    if (!fgets(line, sizeof line, f)) return sp3::E_FORMAT;
    std::string banner(line);
    info->pattern = banner.find("pattern") != std::string::npos;
    info->symm = banner.find("symmetric") != std::string::npos;
    info->cplx = banner.find("complex") != std::string::npos;
    // a first line that is not a banner is treated as the size line
    bool have_size = false;
    if (banner.empty() || banner[0] != '%') {
        have_size = sscanf(line, "%lu %lu %lu", &info->nrows, &info->ncols, &info->file_nnz) == 3;
        if (!have_size) return sp3::E_FORMAT;
    }
    while (!have_size) {
        if (!fgets(line, sizeof line, f)) return sp3::E_FORMAT;
        if (line[0] == '%') continue;
        char* p = line; while (*p == ' ' || *p == '\t') ++p;
        if (*p == '\n' || *p == 0 || *p == '\r') continue;
        if (sscanf(line, "%lu %lu %lu", &info->nrows, &info->ncols, &info->file_nnz) != 3) return sp3::E_FORMAT;
        have_size = true;
    }
    info->data_off = ftell(f);
    return sp3::OK;
}
}  // namespace

// flags bit0 = pattern, bit1 = symmetric, bit2 = complex.  max_nnz is the
// capacity the caller must provide to sp3_mm_read (2x for symmetric files).
SP3_API int sp3_mm_read_header(const char* path, uint64_t* nrows, uint64_t* ncols,
                               uint64_t* file_nnz, uint64_t* max_nnz, int* flags) {
    FILE* f = fopen(path, "r");
    if (!f) return sp3::E_IO;
    MMInfo info{};
    int rc = mm_parse_header(f, &info);
    fclose(f);
    if (rc != sp3::OK) return rc;
    *nrows = info.nrows; *ncols = info.ncols; *file_nnz = info.file_nnz;
    *max_nnz = info.symm ? 2 * info.file_nnz : info.file_nnz;
    *flags = (info.pattern ? 1 : 0) | (info.symm ? 2 : 0) | (info.cplx ? 4 : 0);
    return sp3::OK;
}

SP3_API int sp3_mm_read(const char* path, uint64_t capacity, int mirror_diagonal,
                        uint32_t* rows, uint32_t* cols, double* vals, uint64_t* nnz_out) {
    FILE* f = fopen(path, "r");
    if (!f) return sp3::E_IO;
    MMInfo info{};
    int rc = mm_parse_header(f, &info);
    if (rc != sp3::OK) { fclose(f); return rc; }
    uint64_t need = info.symm ? 2 * info.file_nnz : info.file_nnz;
    if (capacity < need) { fclose(f); return sp3::E_CAPACITY; }
    // slurp the data section and parse with strtoul/strtod (fast, locale free)
    fseek(f, 0, SEEK_END);
    long end = ftell(f);
    fseek(f, info.data_off, SEEK_SET);
    std::vector<char> text((size_t)(end - info.data_off) + 1);
    size_t got = fread(text.data(), 1, text.size() - 1, f);
    text[got] = 0;
    fclose(f);
    char* p = text.data();
    uint64_t n = 0, mirrored = 0;
    const uint64_t half = info.file_nnz;
    for (uint64_t i = 0; i < info.file_nnz; ++i) {
        char* q;
        unsigned long r = strtoul(p, &q, 10);
        if (q == p) return sp3::E_FORMAT;
        p = q;
        unsigned long c = strtoul(p, &q, 10);
        if (q == p) return sp3::E_FORMAT;
        p = q;
        double v = 1.0;
        if (!info.pattern) {
            v = strtod(p, &q);
            if (q == p) return sp3::E_FORMAT;
            p = q;
            if (info.cplx) { strtod(p, &q); if (q == p) return sp3::E_FORMAT; p = q; }
        }
        if (r < 1 || c < 1 || r > info.nrows || c > info.ncols) return sp3::E_RANGE;
        rows[n] = (uint32_t)(r - 1); cols[n] = (uint32_t)(c - 1); vals[n] = v;
        if (info.symm && (mirror_diagonal || r != c)) {
            // mirrored copies live in the second half, in file order
            rows[half + mirrored] = (uint32_t)(c - 1);
            cols[half + mirrored] = (uint32_t)(r - 1);
            vals[half + mirrored] = v;
            ++mirrored;
        }
        ++n;
    }
    *nnz_out = n + mirrored;
    return sp3::OK;
}

// Writes a general real coordinate MatrixMarket file (1-based), used by tests
// and by the CLI tools to hand matrices to other programs.
SP3_API int sp3_mm_write(const char* path, uint64_t nrows, uint64_t ncols, uint64_t nnz,
                         const uint32_t* rows, const uint32_t* cols, const double* vals) {
    FILE* f = fopen(path, "w");
    if (!f) return sp3::E_IO;
    fprintf(f, "%%%%MatrixMarket matrix coordinate real general\n%lu %lu %lu\n", nrows, ncols, nnz);
    for (uint64_t i = 0; i < nnz; ++i)
        fprintf(f, "%u %u %.17g\n", rows[i] + 1, cols[i] + 1, vals ? vals[i] : 1.0);
    return fclose(f) == 0 ? sp3::OK : sp3::E_IO;
}

// Shared declarations for the native host library (libsp3host.so).
//
// Every exported function is `extern "C"`, takes caller-allocated arrays and
// returns 0 on success or a negative error code; sizes that are not known in
// advance are obtained with a counting call first.  Index type on disk and in
// the partitioning code is u32 (the reference's idx_t, src/basic.hpp:16-18),
// nnz counts are 64-bit.
#pragma once
#include <cstdint>
#include <cstddef>

#define SP3_API extern "C" __attribute__((visibility("default")))

namespace sp3 {

// Counter-based RNG: every random decision is a pure function of
// (seed, stream, index), so results do not depend on thread count or on the
// order ranks make their calls.
static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline uint64_t rnd(uint64_t seed, uint64_t stream, uint64_t idx) {
    return mix64(mix64(seed ^ (stream * 0xD6E8FEB86659FD93ull)) + idx * 0x9E3779B97F4A7C15ull);
}
static inline double u01(uint64_t bits) {  // uniform in [0,1)
    return (double)(bits >> 11) * (1.0 / 9007199254740992.0);
}
// Standard normal from two counter draws (Box-Muller).
double normal01(uint64_t seed, uint64_t stream, uint64_t idx);

enum Err : int {
    OK = 0,
    E_IO = -1,
    E_FORMAT = -2,
    E_RANGE = -3,
    E_ARG = -4,
    E_CAPACITY = -5,
};

}  // namespace sp3

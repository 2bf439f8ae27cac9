// Common device helpers for the sm_100a kernels of libsp3cuda.so.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#define SP3_API extern "C" __attribute__((visibility("default")))

namespace sp3 {

// ---- status word -----------------------------------------------------------
// Kernels never trap.  A kernel that meets a bad index or a wait that runs out
// writes one record into a caller-provided int32[4] status array
// {code, detail0, detail1, detail2} (first writer wins) and returns normally;
// the host reads it after synchronising.
enum StatusCode : int {
    ST_OK = 0,
    ST_BAD_INDEX = 1,      // detail0 = which array, detail1 = position, detail2 = value
    ST_WAIT_TIMEOUT = 2,   // detail0 = wait site, detail1 = peer / tile, detail2 = observed value
};

__device__ __forceinline__ void report(int* status, int code, int d0, int d1, int d2) {
    if (status && atomicCAS(status, 0, code) == 0) {
        status[1] = d0; status[2] = d1; status[3] = d2;
        __threadfence_system();
    }
}

// ---- 16-byte vector access -------------------------------------------------
template <typename T> struct Vec;
template <> struct Vec<float> { using type = float4; static constexpr int N = 4; };
template <> struct Vec<double> { using type = double2; static constexpr int N = 2; };

__device__ __forceinline__ float4 vzero(float4*) { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ double2 vzero(double2*) { return make_double2(0.0, 0.0); }
__device__ __forceinline__ float vdot(const float4& a, const float4& b) {
    return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
}
__device__ __forceinline__ double vdot(const double2& a, const double2& b) { return a.x * b.x + a.y * b.y; }
__device__ __forceinline__ void vfma(float4& acc, float s, const float4& x) {
    acc.x += s * x.x; acc.y += s * x.y; acc.z += s * x.z; acc.w += s * x.w;
}
__device__ __forceinline__ void vfma(double2& acc, double s, const double2& x) { acc.x += s * x.x; acc.y += s * x.y; }
__device__ __forceinline__ void vadd(float4& acc, const float4& x) { acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w; }
__device__ __forceinline__ void vadd(double2& acc, const double2& x) { acc.x += x.x; acc.y += x.y; }
__device__ __forceinline__ float4 vscale(float s, const float4& x) { return make_float4(s * x.x, s * x.y, s * x.z, s * x.w); }
__device__ __forceinline__ double2 vscale(double s, const double2& x) { return make_double2(s * x.x, s * x.y); }

__device__ __forceinline__ float4 shfl_xor_vec(const float4& v, int m) {
    return make_float4(__shfl_xor_sync(0xffffffffu, v.x, m), __shfl_xor_sync(0xffffffffu, v.y, m),
                       __shfl_xor_sync(0xffffffffu, v.z, m), __shfl_xor_sync(0xffffffffu, v.w, m));
}
__device__ __forceinline__ double2 shfl_xor_vec(const double2& v, int m) {
    return make_double2(__shfl_xor_sync(0xffffffffu, v.x, m), __shfl_xor_sync(0xffffffffu, v.y, m));
}

// ---- system-scope flags over NVLink ----------------------------------------
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Spins until *flag >= want (acquire, system scope) or `limit_ns` passes.
// Returns true on success.  Never spins without a bound.
__device__ __forceinline__ bool wait_ge_sys(const int* flag, int want, unsigned long long limit_ns, int* seen) {
    int v = ld_acquire_sys(flag);
    if (v >= want) { *seen = v; return true; }
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i) {
            v = ld_acquire_sys(flag);
            if (v >= want) { *seen = v; return true; }
            __nanosleep(64);
        }
        if (globaltimer_ns() - t0 > limit_ns) { *seen = v; return false; }
    }
}
__device__ __forceinline__ bool wait_ge_gpu(const int* flag, int want, unsigned long long limit_ns, int* seen) {
    int v = ld_acquire_gpu(flag);
    if (v >= want) { *seen = v; return true; }
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i) {
            v = ld_acquire_gpu(flag);
            if (v >= want) { *seen = v; return true; }
            __nanosleep(32);
        }
        if (globaltimer_ns() - t0 > limit_ns) { *seen = v; return false; }
    }
}

// read-only load of a pointer-table entry
template <typename P> __device__ __forceinline__ P* ldg_ptr(P* const* slot) {
    return reinterpret_cast<P*>(__ldg(reinterpret_cast<const unsigned long long*>(slot)));
}

// lanes-per-row choice: smallest power of two G (<= 32) with G * VN >= k,
// R = vectors per lane.
__host__ __device__ inline int pick_group(int nvec) {
    int g = 1;
    while (g < 32 && g < nvec) g <<= 1;
    return g;
}

}  // namespace sp3

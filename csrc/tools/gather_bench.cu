// gather_bench: how fast can one B200 gather random dense rows, with vector loads and with the asynchronous
// copy unit?
//
//   gather_bench [log2 of the table rows, default 21]
//
// The local SDDMM and SpMM kernels spend their time fetching one dense row (k * 4 bytes) per nonzero.  This
// programme measures that access pattern alone, for k = 32 ... 256:
//   lsu   lane groups fetch rows with 16-byte vector loads, four rows in flight per group (the inner loop of
//         the local kernels without the arithmetic);
//   bulk  P producer warps issue one `cp.async.bulk` per row into a shared-memory ring (mbarrier completion),
//         the other warps read the rows from shared memory.
// A table of 2^21 rows does not fit the L2 cache (device-memory rate), 2^16 rows do (L2 rate).  The figures
// decide which engine the kernels use: measured on B200, vector loads deliver 25-28 B/clk/SM from device memory
// and 57-67 B/clk/SM from L2, the copy unit at most one row every 14-16 clocks per SM whatever its size
// (35 B/clk/SM for 512-byte rows from L2, 8-11 for 128-byte rows).  Rows of a kilobyte or less are therefore
// gathered with vector loads; the copy unit is used where its asynchrony pays, for pulling rows over NVLink
// (fused_impl.cuh).  The reference has no counterpart (its loops are scalar, src/core_ops.cpp:5-35).
//
// Built by spcomm3d_b200.utils.native.build_tools() into spcomm3d_b200/_lib/gather_bench.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime.h>
#include "sp3_async.cuh"
using namespace sp3;

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)

// ---- LSU gather: lane groups of G lanes x R float4 per row, U rows in flight per group
template <int G, int R, int U>
__global__ void __launch_bounds__(256, 4) lsu_gather(const float4* __restrict__ tab, long long ld_v, const int* __restrict__ idx,
                                                     long long n, float* out) {
    const int lane = threadIdx.x & 31, slot = lane / G, gl = lane % G;
    constexpr int SLOTS = 32 / G;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    float acc = 0.f;
    for (long long base = warp * SLOTS * 32; base < n; base += nwarps * SLOTS * 32) {
        const long long b0 = base + slot * 32;
        for (int j = 0; j < 32; j += U) {
            float4 v[U][R];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long i = b0 + j + u;
                const int r = i < n ? __ldg(idx + i) : 0;
#pragma unroll
                for (int q = 0; q < R; ++q) v[u][q] = __ldg(tab + (long long)r * ld_v + gl + q * G);
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int q = 0; q < R; ++q) acc += v[u][q].x + v[u][q].y + v[u][q].z + v[u][q].w;
        }
    }
    if (acc == 123.456f) out[0] = acc;
}

// ---- bulk gather: warp 0 produces (one cp.async.bulk per row), the other warps consume from shared memory
constexpr int ROWS_PER_STAGE = 32;
template <int STAGES, int P>
__global__ void __launch_bounds__(512, 1) bulk_gather(const float4* __restrict__ tab, long long ld_v, int nvec,
                                                      const int* __restrict__ idx, long long n, float* out, int* err) {
    extern __shared__ __align__(128) unsigned char smem[];
    const unsigned row_bytes = nvec * 16u, stage_bytes = ROWS_PER_STAGE * row_bytes;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + (size_t)STAGES * stage_bytes);
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, ncons = (blockDim.x >> 5) - P;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, ncons); }
        mbar_init_fence();
    }
    __syncthreads();
    const long long per_block = (n / ROWS_PER_STAGE + gridDim.x - 1) / gridDim.x;   // batches per block
    const long long q0 = (long long)blockIdx.x * per_block;
    long long q1 = q0 + per_block; if (q1 > n / ROWS_PER_STAGE) q1 = n / ROWS_PER_STAGE;
    if (wid < P) {
        for (long long q = q0 + wid; q < q1; q += P) {
            const int s = (int)((q - q0) % STAGES);
            const unsigned par = (unsigned)(((q - q0) / STAGES) & 1);
            if (q - q0 >= STAGES && !mbar_wait(empty0 + 8u * s, par ^ 1u)) { *err = 1; return; }
            const int r = __ldg(idx + q * ROWS_PER_STAGE + lane);
            if (lane == 0) mbar_expect_tx(full0 + 8u * s, stage_bytes);
            __syncwarp();
            bulk_load(smem_u32(smem) + s * stage_bytes + lane * row_bytes, tab + (long long)r * ld_v, row_bytes, full0 + 8u * s);
        }
    } else {
        float acc = 0.f;
        const int c = wid - P;
        for (long long q = q0; q < q1; ++q) {
            const int s = (int)((q - q0) % STAGES);
            const unsigned par = (unsigned)(((q - q0) / STAGES) & 1);
            if (!mbar_wait(full0 + 8u * s, par)) { *err = 2; return; }
            // every consumer warp sums its share of the stage (float4 per lane, conflict-free)
            const float4* st = reinterpret_cast<const float4*>(smem + (size_t)s * stage_bytes);
            const int nv = ROWS_PER_STAGE * nvec;
            for (int e = c * 32 + lane; e < nv; e += ncons * 32) { const float4 v = st[e]; acc += v.x + v.y + v.z + v.w; }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8u * s);
        }
        if (acc == 123.456f) out[0] = acc;
    }
}

int main(int argc, char** argv) {
    printf("table rows 2^%d\n", argc > 1 ? atoi(argv[1]) : 21);
    const long long nrows = 1ll << (argc > 1 ? atoi(argv[1]) : 21);   // table rows
    const long long n = 1 << 24;                   // gathered rows per launch
    int clk = 0; CK(cudaDeviceGetAttribute(&clk, cudaDevAttrClockRate, 0));
    int sms = 0; CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
    std::vector<int> h(n);
    unsigned long long x = 88172645463325252ull;
    for (long long i = 0; i < n; ++i) { x ^= x << 13; x ^= x >> 7; x ^= x << 17; h[i] = (int)(x % nrows); }
    int* idx; float* out; int* err; float4* tab;
    CK(cudaMalloc(&idx, n * 4)); CK(cudaMemcpy(idx, h.data(), n * 4, cudaMemcpyHostToDevice));
    CK(cudaMalloc(&out, 4)); CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4));
    CK(cudaMalloc(&tab, nrows * 1024)); CK(cudaMemset(tab, 0, nrows * 1024));
    cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
    for (int k : {32, 64, 128, 256}) {
        const int nvec = k / 4; const long long ld_v = nvec;
        auto report = [&](const char* name, float ms) {
            const double bytes = (double)n * k * 4;
            printf("k=%3d %-22s %.3f ms  %.1f GB/s  %.1f B/clk/SM (at max clock %d MHz)\n", name ? k : k, name, ms, bytes / ms / 1e6,
                   bytes / (ms * 1e-3) / sms / (clk * 1e3), clk / 1000);
        };
        for (int rep = 0; rep < 2; ++rep) {
            cudaEventRecord(a);
            if (k == 32) lsu_gather<8, 1, 4><<<sms * 4, 256>>>(tab, ld_v, idx, n, out);
            if (k == 64) lsu_gather<16, 1, 4><<<sms * 4, 256>>>(tab, ld_v, idx, n, out);
            if (k == 128) lsu_gather<16, 2, 4><<<sms * 4, 256>>>(tab, ld_v, idx, n, out);
            if (k == 256) lsu_gather<16, 4, 4><<<sms * 4, 256>>>(tab, ld_v, idx, n, out);
            cudaEventRecord(b); CK(cudaEventSynchronize(b));
            float ms; cudaEventElapsedTime(&ms, a, b);
            if (rep) report("lsu (4 rows in flight)", ms);
        }
        auto run_bulk = [&](auto kern, int stages, const char* name) {
            const size_t smem = (size_t)stages * ROWS_PER_STAGE * nvec * 16 + 2 * stages * 8 + 64;
            CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            for (int rep = 0; rep < 2; ++rep) {
                cudaEventRecord(a);
                kern<<<sms, 512, smem>>>(tab, ld_v, nvec, idx, n, out, err);
                cudaEventRecord(b); CK(cudaEventSynchronize(b));
                float ms; cudaEventElapsedTime(&ms, a, b);
                if (rep) report(name, ms);
            }
        };
        if ((size_t)8 * ROWS_PER_STAGE * nvec * 16 < 200000) {
            run_bulk(bulk_gather<8, 1>, 8, "bulk 8 stages P=1");
            run_bulk(bulk_gather<8, 2>, 8, "bulk 8 stages P=2");
            run_bulk(bulk_gather<8, 4>, 8, "bulk 8 stages P=4");
            run_bulk(bulk_gather<8, 8>, 8, "bulk 8 stages P=8");
        } else {
            run_bulk(bulk_gather<4, 1>, 4, "bulk 4 stages P=1");
            run_bulk(bulk_gather<4, 2>, 4, "bulk 4 stages P=2");
            run_bulk(bulk_gather<4, 4>, 4, "bulk 4 stages P=4");
        }
    }
    int herr = 0; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
    printf("err=%d\n", herr);
    return 0;
}

// Dense-panel SDDMM on the 5th-generation tensor cores (sm_100a, TF32).
//
// Where the nonzeros of a block of 128 consecutive local rows concentrate in a
// few columns (hub rows x hub columns of a power-law matrix), the block is
// cheaper as a small dense product than as a list of gathers: one CTA stages
// the 128 A rows and the N panel B rows in shared memory, a single thread
// issues `tcgen05.mma.cta_group::1.kind::tf32` over the k dimension with the
// 128 x N fp32 accumulator in tensor memory (TMEM), the tile is read back with
// `tcgen05.ld`, and only the positions that are nonzeros of S are kept:
//   out[pos] = sval * D[row_in_block][column_slot].
// The reference computes every nonzero with a scalar loop
// (src/core_ops.cpp:5-22); this path has no counterpart there.
//
// Operands are rounded to TF32 by the tensor core (10-bit mantissa), so the
// path is opt-in and tested with a matching tolerance.
//
// Shared-memory operand layout (K-major, no swizzle): 16-byte chunk c (4
// floats of k) of row r lives at byte (c * (ROWS + 1) + r) * 16.  A core
// matrix (8 rows x 16 B) is 128 contiguous bytes; the next 8 rows are SBO =
// 128 B away, the next k chunk LBO = (ROWS + 1) * 16 B away (the extra 16 B per
// chunk keep the staging stores of a warp, which writes one row = 32 chunks at
// a time, on distinct banks).  One MMA consumes 8 floats of k (two chunks).
// The accumulator tile is staged for sampling in the space of the A operand,
// which is dead once the MMAs have completed.
#include "sp3_cuda.cuh"

namespace sp3 {

constexpr int PANEL_M = 128;   // rows per panel (TMEM lanes)
constexpr int PANEL_N = 64;    // columns per panel (TMEM columns)
constexpr unsigned PANEL_WAIT_TRIES = 1u << 22;

// bytes of the A operand space: [k/4 chunks][129] float4, at least the 128 x 65 fp32 accumulator staging tile
__host__ __device__ inline size_t panel_a_bytes(int k) {
    const size_t a = (size_t)(k / 4) * (PANEL_M + 1) * 16, d = (size_t)PANEL_M * (PANEL_N + 1) * 4;
    return ((a > d ? a : d) + 127) / 128 * 128;
}

__device__ __forceinline__ unsigned p_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// K-major, SWIZZLE_NONE shared-memory matrix descriptor (version 1 = Blackwell).
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);        // start address, bits [0,14)
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;   // leading byte offset, bits [16,30)
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;   // stride byte offset, bits [32,46)
    d |= 1ull << 46;                                               // descriptor version, bits [46,48)
    return d;                                                      // base offset 0, layout type 0 (no swizzle)
}

// Instruction descriptor: D = F32, A = B = TF32, both K-major, M x N tile.
__host__ __device__ constexpr unsigned umma_idesc_tf32(int M, int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
}

// Resident CTAs per SM of a panel kernel (128 threads, 64 registers): bounded by shared memory (227 KB per SM,
// 1 KB reserved per CTA), by the 512 TMEM columns of an SM and by registers.  Computed here because the
// occupancy query of the runtime answered 1 for these kernels where the hardware fits 2-3.
inline int panel_ctas_per_sm(size_t smem, unsigned tmem_cols) {
    int n = (int)((227u * 1024u) / (smem + 1024));
    const int by_tmem = 512 / (int)tmem_cols;
    if (n > by_tmem) n = by_tmem;
    if (n > 8) n = 8;
    return n < 1 ? 1 : n;
}

__global__ void __launch_bounds__(128)
sddmm_panel_kernel(int npanels, const int* __restrict__ panel_row0, const int* __restrict__ panel_cols,
                   const int* __restrict__ panel_ptr, const unsigned char* __restrict__ e_row,
                   const unsigned char* __restrict__ e_col, const int* __restrict__ e_pos,
                   const float* __restrict__ e_sval, const float* __restrict__ A, long long lda, int nrows_a,
                   const float* __restrict__ B, long long ldb, int k, float* __restrict__ out, int* status) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int nchunk = k / 4;
    constexpr int LDA_S = PANEL_M + 1, LDB_S = PANEL_N + 1;                     // chunk strides in float4
    const size_t a_bytes = panel_a_bytes(k);
    float4* sA = reinterpret_cast<float4*>(smem);                               // [nchunk][129]
    float* sD = reinterpret_cast<float*>(smem);                                 // [128][65], reuses the A space
    float4* sB = reinterpret_cast<float4*>(smem + a_bytes);                     // [nchunk][65]
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(smem + a_bytes + (size_t)nchunk * LDB_S * 16);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bar + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned bar_addr = p_smem_u32(bar);

    if (tid == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_addr));
    if (warp == 0) {  // one warp allocates the accumulator columns and gives up the permit
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(p_smem_u32(tmem_slot)), "r"(PANEL_N));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = *tmem_slot;
    unsigned phase = 0;
    bool ok = true;

    for (int p = blockIdx.x; p < npanels && ok; p += gridDim.x) {
        const int r0 = panel_row0[p];
        // stage the 128 A rows and the 64 panel B rows: a warp reads one row per step, lane = 16-byte chunk
        // (coalesced), four rows in flight
        for (int rr = warp * 32; rr < warp * 32 + 32; rr += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int row = r0 + rr + u;
                const float4* src = reinterpret_cast<const float4*>(A + (long long)(row < nrows_a ? row : r0) * lda);
                v[u] = lane < nchunk ? __ldg(src + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (lane < nchunk) sA[(size_t)lane * LDA_S + rr + u] = v[u];
        }
        for (int rr = warp * 16; rr < warp * 16 + 16; rr += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4* src = reinterpret_cast<const float4*>(B + (long long)panel_cols[(size_t)p * PANEL_N + rr + u] * ldb);
                v[u] = lane < nchunk ? __ldg(src + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (lane < nchunk) sB[(size_t)lane * LDB_S + rr + u] = v[u];
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
        __syncthreads();
        if (tid == 0) {
            const unsigned a0 = p_smem_u32(sA), b0 = p_smem_u32(sB);
            const unsigned idesc = umma_idesc_tf32(PANEL_M, PANEL_N);
            for (int s = 0; s < k / 8; ++s) {  // 8 floats of k = two 16-byte chunks per MMA
                const unsigned long long da = umma_desc(a0 + (unsigned)s * 2u * LDA_S * 16u, LDA_S * 16u, 128u);
                const unsigned long long db = umma_desc(b0 + (unsigned)s * 2u * LDB_S * 16u, LDB_S * 16u, 128u);
                const unsigned acc = s > 0;
                asm volatile(
                    "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                    " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
                    :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
        }
        // bounded wait for the accumulator
        {
            unsigned done = 0;
            for (unsigned i = 0; i < PANEL_WAIT_TRIES && !done; ++i)
                asm volatile("{\n .reg .pred q;\n mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n selp.u32 %0, 1, 0, q;\n}\n"
                             : "=r"(done) : "r"(bar_addr), "r"(phase) : "memory");
            if (!done) { report(status, ST_WAIT_TIMEOUT, 300, p, 0); ok = false; }
            phase ^= 1;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            // warp w reads TMEM lanes 32w..32w+31 (= rows), 32 columns per load
#pragma unroll
            for (int c0 = 0; c0 < PANEL_N; c0 += 32) {
                unsigned v[32];
                const unsigned taddr = tmem_d + ((unsigned)(warp * 32) << 16) + (unsigned)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; ++j) sD[(size_t)tid * (PANEL_N + 1) + c0 + j] = __uint_as_float(v[j]);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (ok)
            for (int e = panel_ptr[p] + tid; e < panel_ptr[p + 1]; e += 128)
                out[e_pos[e]] = e_sval[e] * sD[(size_t)e_row[e] * (PANEL_N + 1) + e_col[e]];
        __syncthreads();  // sD, sA, sB are reused by the next panel
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(PANEL_N));
}


// ---------------------------------------------------------------------------
// Dense-panel SpMM: Y[128 rows of a block] += S_panel (128 x 64, TF32) * X[64 panel columns] (64 x k).
//
// The sparse tile is written out densely in shared memory (zero fill + scatter of the panel's nonzeros) as the
// A operand (M = 128 rows, K = 64 column slots, K-major); the 64 X rows are staged transposed as the B operand
// (N = k features, K = 64 column slots, K-major: chunk c = 4 column slots of feature n at float4 index
// c * (k + 1) + n -- the odd chunk stride makes the transposing stores of a warp, lane = column slot, hit 32
// distinct banks).  The panels of one row block are cut into groups; the panels of a group accumulate into the
// same 128 x k TMEM tile (8 MMAs of K = 8 per panel); after the last one every thread reads its row back with
// `tcgen05.ld` and adds it to Y -- with plain stores when the row block has a single group, with vector atomic
// adds when a hub block was cut into several groups that run on different CTAs.  The nonzeros outside panels run
// through the scheduled gather kernel before this kernel (which also applies beta).
// The reference has one scalar loop for everything (src/core_ops.cpp:24-35).
// ---------------------------------------------------------------------------
constexpr int SPANEL_K = PANEL_N;               // column slots per panel = K of the product
constexpr int SPANEL_CHUNKS = SPANEL_K / 4;     // 16-byte chunks of K
constexpr int LDS_S = PANEL_M + 1;              // chunk stride of the S tile in float4

__host__ __device__ inline size_t spanel_s_bytes() { return ((size_t)SPANEL_CHUNKS * LDS_S * 16 + 127) / 128 * 128; }
__host__ __device__ inline size_t spanel_x_bytes(int k) { return ((size_t)SPANEL_CHUNKS * (k + 1) * 16 + 127) / 128 * 128; }
__host__ __device__ inline unsigned spanel_tmem_cols(int k) { return k <= 32 ? 32u : k <= 64 ? 64u : k <= 128 ? 128u : 256u; }

__global__ void __launch_bounds__(128)
spmm_panel_kernel(int ngroups, const int* __restrict__ grp_ptr, const unsigned char* __restrict__ grp_shared,
                  const int* __restrict__ panel_row0,
                  const int* __restrict__ panel_cols, const int* __restrict__ panel_ptr,
                  const unsigned char* __restrict__ e_row, const unsigned char* __restrict__ e_col,
                  const float* __restrict__ e_sval, const float* __restrict__ X, long long ldx, int k,
                  float* __restrict__ Y, long long ldy, int nrows_y, int* status) {
    extern __shared__ __align__(128) unsigned char smem[];
    float4* sS = reinterpret_cast<float4*>(smem);                                   // [16][129]
    float* sSf = reinterpret_cast<float*>(smem);
    float* sXf = reinterpret_cast<float*>(smem + spanel_s_bytes());                 // [16][k + 1] float4
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(smem + spanel_s_bytes() + spanel_x_bytes(k));
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bar + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned bar_addr = p_smem_u32(bar);
    const unsigned ncols = spanel_tmem_cols(k);
    const int nchunk = k / 4, ldx_s = k + 1;

    if (tid == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_addr));
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(p_smem_u32(tmem_slot)), "r"(ncols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = *tmem_slot;
    unsigned phase = 0;
    bool ok = true;

    for (int g = blockIdx.x; g < ngroups && ok; g += gridDim.x) {
        const int p_begin = grp_ptr[g], p_end = grp_ptr[g + 1];
        const int r0 = panel_row0[p_begin];
        for (int p = p_begin; p < p_end && ok; ++p) {
            // S tile: zero, then scatter the panel's nonzeros (unique positions)
            for (int i = tid; i < SPANEL_CHUNKS * LDS_S; i += 128) sS[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            __syncthreads();
            for (int e = panel_ptr[p] + tid; e < panel_ptr[p + 1]; e += 128) {
                const int r = e_row[e], c = e_col[e];
                sSf[((c >> 2) * LDS_S + r) * 4 + (c & 3)] = e_sval[e];
            }
            // X tile, transposed: lane = column slot of a half, a warp walks its quarter of the feature chunks
            const int cpw = (nchunk + 3) / 4;  // chunks per warp
            const int q_end = (warp + 1) * cpw < nchunk ? (warp + 1) * cpw : nchunk;
            const float4* src[2];
            float* dstj[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int j = half * 32 + lane;
                src[half] = reinterpret_cast<const float4*>(X + (long long)panel_cols[(size_t)p * PANEL_N + j] * ldx);
                dstj[half] = sXf + (size_t)(j >> 2) * ldx_s * 4 + (j & 3);
            }
            for (int q0 = warp * cpw; q0 < q_end; q0 += 4) {  // eight 16-byte loads in flight per lane
                float4 v[2][4];
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        v[half][u] = q0 + u < q_end ? __ldg(src[half] + q0 + u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (q0 + u < q_end) {
                            float* d = dstj[half] + (size_t)(q0 + u) * 16;  // feature 4 * (q0 + u) + i at float 16 * (q0 + u) + 4 * i
                            d[0] = v[half][u].x; d[4] = v[half][u].y; d[8] = v[half][u].z; d[12] = v[half][u].w;
                        }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            if (tid == 0) {
                const unsigned a0 = p_smem_u32(sS), b0 = p_smem_u32(sXf);
                const unsigned idesc = umma_idesc_tf32(PANEL_M, k);
                for (int s = 0; s < SPANEL_K / 8; ++s) {
                    const unsigned long long da = umma_desc(a0 + (unsigned)s * 2u * LDS_S * 16u, LDS_S * 16u, 128u);
                    const unsigned long long db = umma_desc(b0 + (unsigned)s * 2u * (unsigned)ldx_s * 16u, (unsigned)ldx_s * 16u, 128u);
                    const unsigned acc = (p > p_begin) || (s > 0);
                    asm volatile(
                        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                        " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
                        :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
            }
            // bounded wait: the tiles may only be overwritten (and the accumulator read) after the MMAs are done
            {
                unsigned done = 0;
                for (unsigned i = 0; i < PANEL_WAIT_TRIES && !done; ++i)
                    asm volatile("{\n .reg .pred q;\n mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n selp.u32 %0, 1, 0, q;\n}\n"
                                 : "=r"(done) : "r"(bar_addr), "r"(phase) : "memory");
                if (!done) { report(status, ST_WAIT_TIMEOUT, 301, p, 0); ok = false; }
                phase ^= 1;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            ok = __syncthreads_and(ok);
        }
        if (ok) {
            // thread = TMEM lane = row of the block; 32 features per load, added to Y
            const int row = r0 + tid;
            for (int c0 = 0; c0 < k; c0 += 32) {
                unsigned v[32];
                const unsigned taddr = tmem_d + ((unsigned)(warp * 32) << 16) + (unsigned)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < nrows_y && grp_shared[g]) {
                    float4* y = reinterpret_cast<float4*>(Y + (long long)row * ldy + c0);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        atomicAdd(y + q, make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                     __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])));
                } else if (row < nrows_y) {
                    float4* y = reinterpret_cast<float4*>(Y + (long long)row * ldy + c0);
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float4 o = y[q];
                        o.x += __uint_as_float(v[4 * q]); o.y += __uint_as_float(v[4 * q + 1]);
                        o.z += __uint_as_float(v[4 * q + 2]); o.w += __uint_as_float(v[4 * q + 3]);
                        y[q] = o;
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(ncols));
}

}  // namespace sp3

using namespace sp3;

// Panels: panel_row0[p] first local A row of the 128-row block, panel_cols[p*64 + j] the local B row of
// column slot j (unused slots: any valid row), entries panel_ptr[p]..panel_ptr[p+1] with (row in block,
// column slot, output position, S value).  k must be a multiple of 8 and at most 128.
// Returns 0, a cudaError_t, or -1 for an unsupported shape.
SP3_API int sp3_cuda_sddmm_panel_f32(int npanels, const int* panel_row0, const int* panel_cols, const int* panel_ptr,
                                     const unsigned char* e_row, const unsigned char* e_col, const int* e_pos,
                                     const float* e_sval, const float* A, long long lda, int nrows_a, const float* B,
                                     long long ldb, int k, float* out, int* status, void* stream) {
    if (npanels == 0) return 0;
    if (k % 8 || k < 8 || k > 128 || lda % 4 || ldb % 4 || (uintptr_t)A % 16 || (uintptr_t)B % 16) return -1;
    const size_t smem = panel_a_bytes(k) + (size_t)(k / 4) * (PANEL_N + 1) * 16 + 16;
    cudaError_t e = cudaFuncSetAttribute(sddmm_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(sddmm_panel_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int per_sm = panel_ctas_per_sm(smem, PANEL_N);
    const int blocks = npanels < sms * per_sm ? npanels : sms * per_sm;
    sddmm_panel_kernel<<<blocks, 128, smem, (cudaStream_t)stream>>>(npanels, panel_row0, panel_cols, panel_ptr, e_row, e_col,
                                                                    e_pos, e_sval, A, lda, nrows_a, B, ldb, k, out, status);
    return (int)cudaGetLastError();
}

// SpMM twin: groups of consecutive panels that share a row block (grp_ptr[ngroups + 1]); every group adds its
// 128 x k product to Y rows panel_row0 .. +127 (rows >= nrows_y are skipped); grp_shared[g] != 0 says that other
// groups add to the same rows (atomic adds).  Y must already hold beta * Y + (the nonzeros outside panels).  k: a multiple of 32, at most 256.  Returns 0, a cudaError_t or -1.
SP3_API int sp3_cuda_spmm_panel_f32(int ngroups, const int* grp_ptr, const unsigned char* grp_shared,
                                    const int* panel_row0, const int* panel_cols,
                                    const int* panel_ptr, const unsigned char* e_row, const unsigned char* e_col,
                                    const float* e_sval, const float* X, long long ldx, int k, float* Y, long long ldy,
                                    int nrows_y, int* status, void* stream) {
    if (ngroups == 0) return 0;
    if (k % 32 || k < 32 || k > 256 || ldx % 4 || ldy % 4 || (uintptr_t)X % 16 || (uintptr_t)Y % 16) return -1;
    const size_t smem = spanel_s_bytes() + spanel_x_bytes(k) + 16;
    cudaError_t e = cudaFuncSetAttribute(spmm_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(spmm_panel_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int per_sm = panel_ctas_per_sm(smem, spanel_tmem_cols(k));
    const int blocks = ngroups < sms * per_sm ? ngroups : sms * per_sm;
    spmm_panel_kernel<<<blocks, 128, smem, (cudaStream_t)stream>>>(ngroups, grp_ptr, grp_shared, panel_row0, panel_cols, panel_ptr, e_row,
                                                                   e_col, e_sval, X, ldx, k, Y, ldy, nrows_y, status);
    return (int)cudaGetLastError();
}

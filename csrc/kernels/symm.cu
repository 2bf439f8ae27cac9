// Symmetric-heap plumbing: device allocations shared between the ranks of one
// node through CUDA IPC, so that kernels can load and store peers' memory over
// NVLink / NVSwitch with ordinary instructions.
//
// The reference moves all data with MPI messages (src/comm.hpp:105-139); this
// file is what takes their place underneath the fused kernels: one allocation
// per rank, its IPC handle published to the other ranks, peers' mappings
// opened once at setup.
#include "sp3_cuda.cuh"

#include <cstring>

SP3_API int sp3_symm_alloc(size_t bytes, void** out) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(p, 0, bytes);
    if (e != cudaSuccess) { cudaFree(p); return (int)e; }
    *out = p;
    return 0;
}

SP3_API int sp3_symm_free(void* p) { return (int)cudaFree(p); }

// handle: 64 bytes (cudaIpcMemHandle_t)
SP3_API int sp3_ipc_get_handle(void* p, void* handle) {
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) return (int)e;
    static_assert(sizeof(h) == 64, "IPC handle is 64 bytes");
    std::memcpy(handle, &h, sizeof h);
    return 0;
}

SP3_API int sp3_ipc_open(const void* handle, void** out) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof h);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    *out = p;
    return 0;
}

SP3_API int sp3_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

SP3_API int sp3_can_access_peer(int dev, int peer, int* out) {
    return (int)cudaDeviceCanAccessPeer(out, dev, peer);
}

SP3_API const char* sp3_cuda_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

// ---------------------------------------------------------------------------
// Bounded wait on a flag, as a kernel of its own: used by the failure tests
// (a flag nobody sets must end in a status record, not in a hang) and by the
// host-side barrier of the symmetric heap.
// ---------------------------------------------------------------------------
__global__ void wait_flag_kernel(const int* flag, int want, unsigned long long limit_ns, int* status) {
    int seen = 0;
    if (!sp3::wait_ge_sys(flag, want, limit_ns, &seen))
        sp3::report(status, sp3::ST_WAIT_TIMEOUT, /*site*/ 100, 0, seen);
}

SP3_API int sp3_cuda_wait_flag(const int* flag, int want, unsigned long long limit_ns, int* status, void* stream) {
    wait_flag_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag, want, limit_ns, status);
    return (int)cudaGetLastError();
}

// Writes `value` (release, system scope) into the same flag slot of every
// listed pad: the signalling half of the barrier.
__global__ void signal_flags_kernel(int* const* pads, int npads, int slot, int value) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < npads) {
        __threadfence_system();
        sp3::st_release_sys(pads[i] + slot, value);
    }
}

SP3_API int sp3_cuda_signal_flags(void* const* pads_dev, int npads, int slot, int value, void* stream) {
    if (npads == 0) return 0;
    signal_flags_kernel<<<(npads + 63) / 64, 64, 0, (cudaStream_t)stream>>>((int* const*)pads_dev, npads, slot, value);
    return (int)cudaGetLastError();
}

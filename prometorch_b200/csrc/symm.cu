// Symmetric memory over CUDA IPC: every rank allocates the same-sized buffer,
// exports a handle, and maps every peer's buffer into its own address space.
// Kernels then read and write peers' memory with ordinary loads and stores
// that travel over NVLink.  This replaces the reference's TCP and /dev/shm
// process groups (torch/distributed/ddp.cpp:84-139, 287-422): the handle
// exchange is the only traffic that goes through the host.
#include "common.cuh"
#include <string.h>

PTB_API int ptb_symm_alloc(size_t bytes, void** ptr, void* handle64) {
    void* p = nullptr;
    PTB_CUDA_OK(cudaMalloc(&p, bytes));
    PTB_CUDA_OK(cudaMemset(p, 0, bytes));
    cudaIpcMemHandle_t h;
    PTB_CUDA_OK(cudaIpcGetMemHandle(&h, p));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    *ptr = p;
    PTB_CUDA_OK(cudaDeviceSynchronize());
    return 0;
}

PTB_API int ptb_symm_open(const void* handle64, void** ptr) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    PTB_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

PTB_API int ptb_symm_close(void* ptr) {
    PTB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return 0;
}

PTB_API int ptb_symm_free(void* ptr) {
    PTB_CUDA_OK(cudaFree(ptr));
    return 0;
}

// Same-process variant (one process driving several GPUs, used by tests): enable peer access.
PTB_API int ptb_enable_peer_access(int dev, int peer) {
    int can = 0;
    PTB_CUDA_OK(cudaDeviceCanAccessPeer(&can, dev, peer));
    if (!can) { ptb_set_error("device %d cannot access peer %d", dev, peer); return -1; }
    int cur = 0;
    PTB_CUDA_OK(cudaGetDevice(&cur));
    PTB_CUDA_OK(cudaSetDevice(dev));
    cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
    cudaSetDevice(cur);
    PTB_CUDA_OK(e);
    return 0;
}

// Device-memory and device-query entry points of the C ABI.
//
// The reference ships these helpers inside each of its DLLs (kernels/nvfp4_gemv.cu:820-835,
// kernels/nvfp4_cuda_v5.cu:424-457); here one shared library exports them once.  Memory returned
// by gpu_malloc is owned by the caller until gpu_free; callers may do byte arithmetic on the
// returned address (the reference's pair fusion does, experiments/_qwen38_p7_pair.py:123).
#include <cstdio>

#include "common.cuh"

extern "C" {

void* gpu_malloc(size_t bytes) {
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        fprintf(stderr, "gpu_malloc(%zu): %s\n", bytes, cudaGetErrorString(e));
        cudaGetLastError();  // do not leave the failure sticky for the next launch check
        return nullptr;
    }
    return p;
}

void gpu_free(void* p) {
    if (p) cudaFree(p);
}

// Synchronous copies; the return value is the cudaError_t as an int (0 on success).
int gpu_memcpy_h2d(void* dst, const void* src, size_t bytes) {
    return (int)cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice);
}

int gpu_memcpy_d2h(void* dst, const void* src, size_t bytes) {
    return (int)cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost);
}

// device -> device (no counterpart in the reference, whose pair fusion stages such copies through
// host memory: experiments/_qwen38_p7_pair.py:107-114).  Synchronous.
int gpu_memcpy_d2d(void* dst, const void* src, size_t bytes) {
    return (int)cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice);
}

int gpu_sync() { return (cudaDeviceSynchronize() == cudaSuccess) ? 0 : (int)cudaErrorUnknown; }

int get_gpu_info(char* name_buf, int buf_size, int* cc_major, int* cc_minor) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) return -1;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return -2;
    if (name_buf && buf_size > 0) {
        int i = 0;
        while (prop.name[i] != '\0' && i < buf_size - 1) {
            name_buf[i] = prop.name[i];
            i++;
        }
        name_buf[i] = '\0';
    }
    if (cc_major) *cc_major = prop.major;
    if (cc_minor) *cc_minor = prop.minor;
    return 0;
}

// ABI version of this library: major * 100 + minor.
int nvfp4_b200_abi_version() { return 100; }

}  // extern "C"

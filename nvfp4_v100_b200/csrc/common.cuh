// Shared device helpers for the NVFP4 (E2M1 nibbles + one E8M0 scale byte per 16 weights) kernels.
//
// Storage format (reference: codec/nvfp4_codec.py:92-125, 196-200):
//   packed[m][k/2] : byte i of a row holds element 2i in its low nibble and element 2i+1 in its
//                    high nibble; nibble = sign<<3 | code, code indexes {0,.5,1,1.5,2,3,4,6}.
//   scales[m][k/16]: value 2^(byte-127) shared by 16 consecutive elements of the row.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

// The public C ABI: every definition of an exported function is compiled against its
// declaration, so an argument list cannot drift from the header unnoticed.
#include "nvfp4_b200.h"

#define NVFP4_BLOCK 16

// Return codes shared by every launcher (reference: kernels/nvfp4_gemv.cu:842-850).
#define NVFP4_OK 0
#define NVFP4_ERR_LAUNCH (-1)
#define NVFP4_ERR_SHAPE (-2)
#define NVFP4_ERR_ALLOC (-3)

namespace nvfp4 {

// E8M0 byte -> fp32 2^(sb-127): the byte is the fp32 exponent field.  Byte 0 therefore yields
// +0.0f (not the subnormal 2^-127) and byte 255 yields +inf, exactly as the reference kernels do
// (kernels/nvfp4_gemv.cu:44-46).
__device__ __forceinline__ float e8m0_to_f32(uint32_t sb) { return __uint_as_float(sb << 23); }

// Four packed bytes (8 E2M1 nibbles) -> four half2 {element 2i, element 2i+1}, using the sm_100a
// hardware conversion.  The conversion is exact: every E2M1 code point is an fp16 value.
__device__ __forceinline__ void e2m1x8_to_half2x4(uint32_t w, uint32_t& h0, uint32_t& h1,
                                                  uint32_t& h2, uint32_t& h3) {
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3)
        : "r"(w));
}

// One packed byte -> half2 {low nibble, high nibble}.
__device__ __forceinline__ uint32_t e2m1x2_to_half2(uint32_t byte) {
    uint32_t h;
    unsigned short s = (unsigned short)(byte & 0xFFu);
    asm("{\n"
        ".reg .b8 lo, hi;\n"
        "mov.b16 {lo, hi}, %1;\n"
        "cvt.rn.f16x2.e2m1x2 %0, lo;\n"
        "}\n"
        : "=r"(h)
        : "h"(s));
    return h;
}

// Streaming 16-byte load for data that is read once (weights): keep it out of L1 and mark it
// evict-first in L2 so it does not displace the activation vector or the scale bytes.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float round_f16(float x) { return __half2float(__float2half(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Attributes set with cudaFuncSetAttribute and device properties hold for ONE device; a process
// may drive several, so the launchers cache such facts per device index.
constexpr int NVFP4_MAX_DEVICES = 64;
static inline int current_device_index() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NVFP4_MAX_DEVICES) dev = 0;
    return dev;
}

// Programmatic dependent launch.  A kernel that starts with pdl_prologue() may be launched with
// the programmatic-stream-serialization attribute: it becomes resident while the previous kernel
// in the stream is still draining, lets ITS successor do the same, and then waits for the
// previous kernel to complete before touching memory.  Without the attribute both are no-ops.
// After the wait, every pointer to memory that an earlier kernel may have written goes through
// PDL_FRESH.  A kernel parameter declared `const T* __restrict__` tells the compiler that the data
// never changes while the kernel runs, so it may issue such a load anywhere - also ABOVE the wait,
// while the previous kernel is still writing (seen: a token id read before the kernel that
// produces it had finished).  An empty asm that "modifies" the pointer makes the value opaque:
// loads through it cannot move above the asm, and are ordinary coherent loads.
#define PDL_FRESH(p) asm volatile("" : "+l"(p))

__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

// Launch with the attribute (kernels that call pdl_prologue() first thing).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace nvfp4

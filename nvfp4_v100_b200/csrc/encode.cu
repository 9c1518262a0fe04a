// fp16 -> NVFP4 quantiser on the device: one thread per 16-element block.
//
// The reference quantises on the CPU (codec/nvfp4_codec.py:166-245; vectorised:
// codec/nvfp4_codec_fast.py:19-53, pipeline/_qwen38_nvfp4_pack.py:34-67) with logarithms and a
// table search in float64.  The same bytes come out of exact integer / fp32 steps:
//   scale : the block maximum is 1.f * 2^E as an fp32 (every fp16 value is a normal fp32); the
//           smallest e with 6 * 2^e >= max is E - 2 when 1.f <= 1.5 and E - 1 otherwise;
//           an all-zero block gets e = 0; byte = e + 127.
//   code  : |x| * 2^-e is exact in fp32 (an 11-bit significand times a power of two); the code is
//           the number of midpoints {0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5} strictly below it, so a
//           value on a midpoint takes the smaller code.  Sign bit only for values below zero.
// Non-finite inputs follow what the CPU arithmetic does with them: a block holding +-inf gets
// byte 254, a block holding a NaN gets byte 127, a NaN element gets code 7.
//
// The kernel is a pure stream: 2 bytes read and 0.5625 bytes written per element.
#include "common.cuh"

namespace nvfp4 {

__device__ __forceinline__ uint32_t e2m1_code_of(float a) {
    uint32_t c = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) +
                 (a > 5.0f);
    return (a != a) ? 7u : c;
}

__global__ void __launch_bounds__(256)
encode_kernel(const uint4* __restrict__ src, uint2* __restrict__ packed,
              uint8_t* __restrict__ scales, long long nblocks) {
    pdl_prologue();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += stride) {
        const uint4 v0 = __ldg(src + 2 * b), v1 = __ldg(src + 2 * b + 1);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        // magnitudes of fp16 values order like their bit patterns (NaN above inf above finite)
        uint32_t mx = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            mx = max(mx, w[i] & 0x7FFFu);
            mx = max(mx, (w[i] >> 16) & 0x7FFFu);
        }
        int e;
        if (mx == 0u) {
            e = 0;
        } else if (mx >= 0x7C00u) {
            e = (mx == 0x7C00u) ? 127 : 0;
        } else {
            const uint32_t fb = __float_as_uint(__half2float(__ushort_as_half((unsigned short)mx)));
            e = (int)(fb >> 23) - 127 - (((fb & 0x7FFFFFu) <= 0x400000u) ? 2 : 1);
        }
        // 2^-e; e = 127 needs the subnormal 2^-127
        const float inv = (e == 127) ? __uint_as_float(0x00400000u)
                                     : __uint_as_float((uint32_t)(127 - e) << 23);
        uint32_t out[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            const float lo = f.x * inv, hi = f.y * inv;
            const uint32_t nlo = e2m1_code_of(fabsf(lo)) | (lo < 0.0f ? 8u : 0u);
            const uint32_t nhi = e2m1_code_of(fabsf(hi)) | (hi < 0.0f ? 8u : 0u);
            out[i >> 2] |= (nlo | (nhi << 4)) << (8 * (i & 3));
        }
        packed[b] = make_uint2(out[0], out[1]);
        scales[b] = (uint8_t)(e + 127);
    }
}

}  // namespace nvfp4

extern "C" {

// src fp16 [M, K] row-major -> packed [M, K/2], scales [M, K/16].  K % 16 == 0; src 16-byte and
// packed 8-byte aligned.  Asynchronous on `stream`, capturable.  0; -2 bad shape / pointer;
// -1 launch error.
int launch_nvfp4_encode(const void* src_fp16, void* packed, void* scales, int M, int K,
                        void* stream) {
    if (M <= 0 || K <= 0 || K % 16 != 0) return NVFP4_ERR_SHAPE;
    if (!src_fp16 || !packed || !scales) return NVFP4_ERR_SHAPE;
    if (((uintptr_t)src_fp16 & 15) || ((uintptr_t)packed & 7)) return NVFP4_ERR_SHAPE;
    const long long nblocks = (long long)M * (K / 16);
    long long want = (nblocks + 255) / 256;
    const long long cap = 148LL * 8 * 4;   // a few waves of 8 CTAs per SM; grid-stride beyond
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    const cudaError_t e = nvfp4::launch_pdl(nvfp4::encode_kernel, dim3(grid), dim3(256), 0,
                                            (cudaStream_t)stream, (const uint4*)src_fp16,
                                            (uint2*)packed, (uint8_t*)scales, nblocks);
    return e == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH;
}

}  // extern "C"

// NVFP4 codec on the device.
//
// Quantiser (fp16 -> NVFP4): one thread per 16-element block.
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

// One byte: low nibble = code of lo, high nibble = code of hi (hardware conversion, see its use).
__device__ __forceinline__ uint32_t e2m1x2_of(float lo, float hi) {
    uint32_t r;
    asm("{\n.reg .b8 b;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n"
        "cvt.u32.u8 %0, b;\n}\n"
        : "=r"(r)
        : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t e2m1_code_of(float a) {
    uint32_t c = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) +
                 (a > 5.0f);
    return (a != a) ? 7u : c;
}

__global__ void __launch_bounds__(256)
encode_kernel(const uint4* __restrict__ src, uint2* __restrict__ packed,
              uint8_t* __restrict__ scales, long long nblocks) {
    // Waits for its predecessor but does NOT let its successor start early: what it writes are
    // weights, and the GEMV requests weights before waiting for the kernel in front of it.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    PDL_FRESH(src);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += stride) {
        const uint4 v0 = src[2 * b], v1 = src[2 * b + 1];
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
        // The code of |x| 2^-e is the hardware conversion's (cvt.rn.satfinite.e2m1x2: round to
        // nearest, ties to the even code, NaN to +6) once ties are out of the way: the rule here is
        // "a value on a midpoint takes the smaller code", the hardware's would take the larger one
        // at 0.75, 1.75 and 3.5.  Scaling by 2^-e (1 - 2^-20) instead of 2^-e moves a midpoint just
        // below itself and no other input across one (|x| 2^-e has 11 significant bits: it is on a
        // midpoint or at least 2^-11 of its size away).  The fused add of +0 turns a -0 product
        // into +0: the sign bit is for values below zero only.
        const float invn = inv * 0.99999904632568359375f;
        uint32_t out[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            const float lo = fmaf(f.x, invn, 0.0f), hi = fmaf(f.y, invn, 0.0f);
            out[i >> 2] |= e2m1x2_of(lo, hi) << (8 * (i & 3));
        }
        packed[b] = make_uint2(out[0], out[1]);
        scales[b] = (uint8_t)(e + 127);
    }
}

// Dequantiser (NVFP4 rows -> fp16): value = code point x 2^(scale byte - 127), one rounding to
// fp16 — what the reference's decoder computes in float64 (codec/nvfp4_codec.py:248-275; the
// vectorised row decoder of its embedding table, pipeline/_qwen38_infer.py:117-128).  A code point
// has 2 significant bits, so the product is exact in fp32 for scale bytes 1..254; byte 0 (2^-127)
// rounds every code point to zero in fp16 and byte 255 (2^128) sends every non-zero one to
// infinity, which the two fix-ups below reproduce.  One thread per 16-element block; rows are
// taken from `ids` (device int64, clamped to the table) or in order when ids is NULL.
__global__ void __launch_bounds__(256)
decode_rows_kernel(const uint2* __restrict__ packed, const uint8_t* __restrict__ scales,
                   const long long* __restrict__ ids, uint4* __restrict__ out, int K,
                   long long table_rows) {
    pdl_prologue();
    PDL_FRESH(packed); PDL_FRESH(scales); PDL_FRESH(ids); PDL_FRESH(out);
    const int nb = K >> 4;
    const int b = blockIdx.x * 256 + threadIdx.x;
    if (b >= nb) return;
    long long row = ids ? ids[blockIdx.y] : (long long)blockIdx.y;
    if (row < 0) row = 0;
    if (row >= table_rows) row = table_rows - 1;
    const uint2 pk = __ldg(packed + (size_t)row * nb + b);
    const uint32_t sb = scales[(size_t)row * nb + b];
    float sc = e8m0_to_f32(sb < 254u ? sb : 254u);
    const float extra = (sb == 255u) ? 2.0f : 1.0f;
    uint32_t h[8];
    e2m1x8_to_half2x4(pk.x, h[0], h[1], h[2], h[3]);
    e2m1x8_to_half2x4(pk.y, h[4], h[5], h[6], h[7]);
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
        const __half2 r = __floats2half2_rn(f.x * sc * extra, f.y * sc * extra);
        o[i] = *reinterpret_cast<const uint32_t*>(&r);
    }
    uint4* dst = out + ((size_t)blockIdx.y * nb + b) * 2;
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// Activation quantisation for a W4A4 product: every 16-element block of a token row is quantised
// exactly as encode_kernel does and immediately dequantised, and the result is written
// token-minor (dst[k][t], rows ld_dst long, columns n .. ld_dst-1 zeroed), the layout the GEMM
// reads.  The values are those a block-scaled FP4 x FP4 tensor-core product would see.  Thread =
// (token, block): consecutive threads take consecutive tokens, so the transposed stores coalesce.
__global__ void __launch_bounds__(256)
quant_dequant_T_kernel(const __half* __restrict__ src, long long ld_src, __half* __restrict__ dst,
                       long long ld_dst, int n) {
    pdl_prologue();
    PDL_FRESH(src); PDL_FRESH(dst);
    const int t = blockIdx.x * 256 + threadIdx.x;
    const int b = blockIdx.y;
    if (t >= ld_dst) return;
    uint32_t w[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    if (t < n) {
        const uint4* p = reinterpret_cast<const uint4*>(src + (size_t)t * ld_src + (size_t)b * 16);
        const uint4 v0 = __ldg(p), v1 = __ldg(p + 1);
        w[0] = v0.x; w[1] = v0.y; w[2] = v0.z; w[3] = v0.w;
        w[4] = v1.x; w[5] = v1.y; w[6] = v1.z; w[7] = v1.w;
    }
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
    const float inv = (e == 127) ? __uint_as_float(0x00400000u)
                                 : __uint_as_float((uint32_t)(127 - e) << 23);
    const float sc = __uint_as_float((uint32_t)(e + 127 < 254 ? e + 127 : 254) << 23);
    __half* col = dst + (size_t)b * 16 * ld_dst + t;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        const float v[2] = {f.x * inv, f.y * inv};
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t c = e2m1_code_of(fabsf(v[u]));
            // code point: 0, .5, 1, 1.5, 2, 3, 4, 6
            const float mag = (c < 4u) ? 0.5f * (float)c : (c == 4u ? 2.0f : (c == 5u ? 3.0f : (c == 6u ? 4.0f : 6.0f)));
            const float q = (v[u] < 0.0f) ? -mag : mag;
            col[(size_t)(2 * i + u) * ld_dst] = __float2half_rn(q * sc);
        }
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

// out[r][0..K) (fp16, 16-byte aligned, rows contiguous) = dequantised row ids[r] of the table
// packed [table_rows][K/2] / scales [table_rows][K/16]; ids: device int64 [n_rows] or NULL for
// rows 0 .. n_rows-1.  K % 16 == 0, packed 8-byte aligned.  0; -2 bad arguments; -1 launch error.
int launch_nvfp4_decode_rows(const void* packed, const void* scales, const void* ids, void* out,
                             int n_rows, int K, long long table_rows, void* stream) {
    if (!packed || !scales || !out || n_rows <= 0 || n_rows > 65535 || K <= 0 || K % 16 != 0 ||
        table_rows <= 0)
        return NVFP4_ERR_SHAPE;
    if (((uintptr_t)packed & 7) || ((uintptr_t)out & 15) || ((uintptr_t)ids & 7))
        return NVFP4_ERR_SHAPE;
    const dim3 grid((K / 16 + 255) / 256, n_rows);
    const cudaError_t e = nvfp4::launch_pdl(nvfp4::decode_rows_kernel, grid, dim3(256), 0,
                                            (cudaStream_t)stream, (const uint2*)packed,
                                            (const uint8_t*)scales, (const long long*)ids,
                                            (uint4*)out, K, table_rows);
    return e == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH;
}

// dst[k][t] (fp16, rows ld_dst >= n long, tail zeroed) = dequantise(quantise(src[t][0..K))), the
// codec applied along K per token row.  K % 16 == 0, src 16-byte aligned, ld_src % 8 == 0.
// 0; -2 bad arguments; -1 launch error.
int launch_nvfp4_quant_dequant_T(const void* src, long long ld_src, void* dst, long long ld_dst,
                                 int n, int K, void* stream) {
    if (!src || !dst || n <= 0 || K <= 0 || K % 16 != 0 || K / 16 > 65535 || ld_src < K ||
        (ld_src & 7) || ld_dst < n || ((uintptr_t)src & 15))
        return NVFP4_ERR_SHAPE;
    const dim3 grid((unsigned)((ld_dst + 255) / 256), K / 16);
    const cudaError_t e = nvfp4::launch_pdl(nvfp4::quant_dequant_T_kernel, grid, dim3(256), 0,
                                            (cudaStream_t)stream, (const __half*)src, ld_src,
                                            (__half*)dst, ld_dst, n);
    return e == cudaSuccess ? NVFP4_OK : NVFP4_ERR_LAUNCH;
}

}  // extern "C"

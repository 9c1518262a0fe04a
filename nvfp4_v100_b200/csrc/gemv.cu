// Batch-1 / batch-2 NVFP4 GEMV for sm_100a:  out[a][m] = sum_k W[m][k] * act_a[k].
//
// Replaces the reference's decode GEMV family (kernels/nvfp4_gemv.cu:499-574 v8 kernel, :659-730
// two-activation kernel, launchers :837-1011).  The reference multiplies in fp16 (8 chained hfma2
// per block); this kernel keeps every product exact and accumulates in fp32.
//
// The kernel is HBM-bound (0.5625 B per weight), so the design goal is: few instructions per
// weight, many bytes in flight, long contiguous reads.
//   * A CTA owns 16 consecutive rows; its warps interleave over 256-wide K steps, so one CTA
//     iteration reads WARPS*128 contiguous bytes of each of the 16 rows.
//   * A lane reads 32 B (64 nibbles = 4 scale blocks) of row g and of row g+8 with one 256-bit
//     evict-first load each, converts nibbles to fp16 with cvt.rn.f16x2.e2m1x2 (exact), and feeds
//     them to mma.sync.m16n8k16 (fp16 x fp16 -> fp32) as the A operand.
//   * The B operand holds the activation only in column n == (lane's K chunk), zero elsewhere, so
//     accumulator column n is the partial sum of exactly one 16-weight scale block of one row.
//     After the 4 MMAs that cover a block the fp32 partial sum is multiplied by the block's
//     2^(sb-127) and added to the row's running fp32 sum.  Columns 4..7 carry the second
//     activation of the batch-2 entry point at no extra weight traffic.
//   * The tensor pipe is used purely as an exact fp16-product / fp32-sum dot-product unit; at one
//     MMA per 256 weights it is far from saturated.
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace nvfp4 {

__device__ __forceinline__ void ld_stream_256(const void* p, uint32_t (&r)[8]) {
    asm volatile(
        "ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7])
        : "l"(p));
}

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// byte q (0..3) of w as an E8M0 scale in fp32
__device__ __forceinline__ float scale_byte(uint32_t w, int q) {
    return __uint_as_float(((w >> (8 * q)) & 0xFFu) << 23);
}

struct WeightRegs {
    uint32_t wa[8];  // 32 packed bytes of row g
    uint32_t wb[8];  // 32 packed bytes of row g+8
    uint2 sa, sb;    // 8 scale bytes of row g / g+8: .x = blocks 0..3 of the even chunk, .y = odd
};

// Tensor-core GEMV.  Requirements checked by the launcher: K % 128 == 0, packed 32-byte aligned,
// scales 8-byte aligned, activations 16-byte aligned.
template <int WARPS, int NACT>
__global__ void __launch_bounds__(WARPS * 32)
gemv_mma_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                const __half* __restrict__ act0, const __half* __restrict__ act1,
                __half* __restrict__ out, int M, int K) {
    __shared__ float red[WARPS][16][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nsteps = (K + 255) >> 8;
    const int ntiles = (M + 15) >> 4;
    const size_t prow = (size_t)(K >> 1), srow = (size_t)(K >> 4);
    // Lane (g,t) supplies column g of B with the activation of K chunk t when (g & 3) == t.
    const bool supplies = ((g & 3) == t) && (g < 4 || NACT == 2);
    const __half* xsrc = (g < 4 || NACT == 1) ? act0 : act1;

    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int ra = min(tile * 16 + g, M - 1);
        const int rb = min(tile * 16 + g + 8, M - 1);
        const uint8_t* pa = packed + (size_t)ra * prow + t * 32;
        const uint8_t* pb = packed + (size_t)rb * prow + t * 32;
        const uint8_t* sa = scales + (size_t)ra * srow + (t & 1) * 8;
        const uint8_t* sb = scales + (size_t)rb * srow + (t & 1) * 8;
        float acc_a = 0.0f, acc_b = 0.0f;

        auto load_w = [&](int s, WeightRegs& w) {
            if (s * 256 + t * 64 < K) {
                ld_stream_256(pa + (size_t)s * 128, w.wa);
                ld_stream_256(pb + (size_t)s * 128, w.wb);
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) { w.wa[i] = 0u; w.wb[i] = 0u; }
            }
            if (s * 256 + (t & 1) * 128 < K) {
                w.sa = __ldg(reinterpret_cast<const uint2*>(sa + (size_t)s * 16));
                w.sb = __ldg(reinterpret_cast<const uint2*>(sb + (size_t)s * 16));
            } else {
                w.sa = make_uint2(0u, 0u);
                w.sb = make_uint2(0u, 0u);
            }
        };

        WeightRegs cur;
        int s = warp;
        if (s < nsteps) load_w(s, cur);
        for (; s < nsteps; s += WARPS) {
            WeightRegs nxt;
            const int sn = s + WARPS;
            if (sn < nsteps) load_w(sn, nxt);

            // activation of this lane's chunk (suppliers only), 64 halves = 32 half2
            uint32_t xr[32];
            const int kc = s * 256 + t * 64;
            if (supplies && kc < K) {
                const uint4* xp = reinterpret_cast<const uint4*>(xsrc + kc);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint4 v = __ldg(xp + i);
                    xr[4 * i + 0] = v.x; xr[4 * i + 1] = v.y;
                    xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) xr[i] = 0u;
            }

#pragma unroll
            for (int q = 0; q < 4; q++) {  // scale block q of every chunk
                float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                    e2m1x8_to_half2x4(cur.wa[2 * q + h], a0, a1, a2, a3);
                    e2m1x8_to_half2x4(cur.wb[2 * q + h], b0, b1, b2, b3);
                    const int xi = 8 * q + 4 * h;
                    mma_f16_16816(c, a0, b0, a1, b1, xr[xi + 0], xr[xi + 1]);
                    mma_f16_16816(c, a2, b2, a3, b3, xr[xi + 2], xr[xi + 3]);
                }
                acc_a = fmaf(c[0], scale_byte(cur.sa.x, q), acc_a);
                acc_a = fmaf(c[1], scale_byte(cur.sa.y, q), acc_a);
                acc_b = fmaf(c[2], scale_byte(cur.sb.x, q), acc_b);
                acc_b = fmaf(c[3], scale_byte(cur.sb.y, q), acc_b);
            }
            if (sn < nsteps) cur = nxt;
        }

        // lanes t=0,1 hold activation 0 (columns 0..3), lanes t=2,3 activation 1 (columns 4..7)
        acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
        acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
        if ((t & 1) == 0) {
            red[warp][g][t >> 1] = acc_a;
            red[warp][g + 8][t >> 1] = acc_b;
        }
        __syncthreads();
        if (threadIdx.x < 16 * NACT) {
            const int r = threadIdx.x & 15, a = threadIdx.x >> 4;
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) v += red[w][r][a];
            const int row = tile * 16 + r;
            if (row < M) out[(size_t)a * M + row] = __float2half(v);
        }
        __syncthreads();
    }
}

// Generic path for shapes or pointers the tensor-core kernel does not take (K % 128 != 0, or
// weaker alignment): one warp per row, 16-byte loads, fp32 FMA.  K % 32 == 0, packed and
// activations 16-byte aligned, scales 2-byte aligned.
template <int NACT>
__global__ void __launch_bounds__(256)
gemv_generic_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                    const __half* __restrict__ act0, const __half* __restrict__ act1,
                    __half* __restrict__ out, int M, int K) {
    const int row = (blockIdx.x * 256 + threadIdx.x) >> 5;
    if (row >= M) return;
    const int lane = threadIdx.x & 31;
    const int nchunks = K >> 5;  // 32 weights = 16 packed bytes = 2 scale blocks
    const uint8_t* prow = packed + (size_t)row * (size_t)(K >> 1);
    const uint8_t* srow = scales + (size_t)row * (size_t)(K >> 4);
    float acc[NACT];
#pragma unroll
    for (int a = 0; a < NACT; a++) acc[a] = 0.0f;
    for (int c = lane; c < nchunks; c += 32) {
        const uint4 pk = ld_stream_u4(prow + (size_t)c * 16);
        const uint32_t sc2 = __ldg(reinterpret_cast<const unsigned short*>(srow + c * 2));
        const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
        for (int a = 0; a < NACT; a++) {
            const uint4* xp = reinterpret_cast<const uint4*>((a == 0 ? act0 : act1) + (size_t)c * 32);
            float blk[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t h[4];
                e2m1x8_to_half2x4(w[j], h[0], h[1], h[2], h[3]);
                const uint4 xv = __ldg(xp + j);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(&h[p]));
                    const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(&xw[p]));
                    blk[j >> 1] = fmaf(wf.x, xf.x, blk[j >> 1]);
                    blk[j >> 1] = fmaf(wf.y, xf.y, blk[j >> 1]);
                }
            }
            acc[a] = fmaf(blk[0], e8m0_to_f32(sc2 & 0xFFu), acc[a]);
            acc[a] = fmaf(blk[1], e8m0_to_f32(sc2 >> 8), acc[a]);
        }
    }
#pragma unroll
    for (int a = 0; a < NACT; a++) {
        const float v = warp_sum(acc[a]);
        if (lane == 0) out[(size_t)a * M + row] = __float2half(v);
    }
}

struct GemvConfig {
    int warps = 0;         // 0 = choose from the shape
    int ctas_per_sm = 0;   // 0 = choose from the occupancy calculator
    int force_generic = 0;
};
static GemvConfig g_cfg;
static int g_num_sms = 0;

static int num_sms() {
    if (g_num_sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_num_sms = n;
    }
    return g_num_sms;
}

template <int WARPS, int NACT>
static cudaError_t launch_mma(const void* packed, const void* scales, const void* a0, const void* a1,
                              void* out, int M, int K, cudaStream_t st) {
    static int occ = 0;  // resident CTAs per SM for this instantiation
    if (occ == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemv_mma_kernel<WARPS, NACT>,
                                                          WARPS * 32, 0) != cudaSuccess || n <= 0)
            n = 4;
        occ = n;
    }
    const int per_sm = g_cfg.ctas_per_sm > 0 ? g_cfg.ctas_per_sm : occ;
    const int ntiles = (M + 15) / 16;
    int grid = num_sms() * per_sm;
    if (grid > ntiles) grid = ntiles;
    gemv_mma_kernel<WARPS, NACT><<<grid, WARPS * 32, 0, st>>>(
        (const uint8_t*)packed, (const uint8_t*)scales, (const __half*)a0, (const __half*)a1,
        (__half*)out, M, K);
    return cudaGetLastError();
}

static inline bool aligned(const void* p, uintptr_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// Shared body of every GEMV entry point.  nact = 1 or 2.
int gemv_dispatch(const void* packed, const void* scales, const void* a0, const void* a1, void* out,
                  int M, int K, void* stream, int nact, const char* who) {
    if (K <= 0 || K % (NVFP4_BLOCK * 2) != 0) return NVFP4_ERR_SHAPE;
    if (M <= 0) return NVFP4_ERR_SHAPE;
    if (!packed || !scales || !a0 || !out || (nact == 2 && !a1)) return NVFP4_ERR_SHAPE;
    if (!aligned(packed, 16) || !aligned(a0, 16) || (nact == 2 && !aligned(a1, 16)) ||
        !aligned(scales, 2) || !aligned(out, 2))
        return NVFP4_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const bool fast = !g_cfg.force_generic && (K % 128 == 0) && aligned(packed, 32) &&
                      aligned(scales, 8);
    if (fast) {
        int warps = g_cfg.warps;
        if (warps == 0) warps = (K >= 8192) ? 8 : 4;
        if (nact == 1) {
            e = (warps == 8) ? launch_mma<8, 1>(packed, scales, a0, a1, out, M, K, st)
              : (warps == 2) ? launch_mma<2, 1>(packed, scales, a0, a1, out, M, K, st)
                             : launch_mma<4, 1>(packed, scales, a0, a1, out, M, K, st);
        } else {
            e = (warps == 8) ? launch_mma<8, 2>(packed, scales, a0, a1, out, M, K, st)
                             : launch_mma<4, 2>(packed, scales, a0, a1, out, M, K, st);
        }
    } else {
        const unsigned grid = (unsigned)((M + 7) / 8);
        if (nact == 1)
            gemv_generic_kernel<1><<<grid, 256, 0, st>>>((const uint8_t*)packed,
                (const uint8_t*)scales, (const __half*)a0, (const __half*)a1, (__half*)out, M, K);
        else
            gemv_generic_kernel<2><<<grid, 256, 0, st>>>((const uint8_t*)packed,
                (const uint8_t*)scales, (const __half*)a0, (const __half*)a1, (__half*)out, M, K);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        fprintf(stderr, "%s launch: %s\n", who, cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return NVFP4_OK;
}

}  // namespace nvfp4

extern "C" {

// Every single-activation GEMV generation of the reference library resolves to the same kernel;
// the names are kept so code written against any of them loads unchanged.
#define NVFP4_GEMV_ENTRY(name)                                                                   \
    int name(const void* weight_packed, const void* weight_scales, const void* activation,       \
             void* output, int M, int K, void* stream) {                                         \
        return nvfp4::gemv_dispatch(weight_packed, weight_scales, activation, nullptr, output,   \
                                    M, K, stream, 1, #name);                                     \
    }
NVFP4_GEMV_ENTRY(launch_nvfp4_gemv)
NVFP4_GEMV_ENTRY(launch_nvfp4_gemv_v8)
NVFP4_GEMV_ENTRY(launch_nvfp4_gemv_v4)
NVFP4_GEMV_ENTRY(launch_nvfp4_gemv_v5)
NVFP4_GEMV_ENTRY(launch_nvfp4_gemv_v6)
NVFP4_GEMV_ENTRY(launch_nvfp4_gemvnl)
#undef NVFP4_GEMV_ENTRY

// The reference's split-K variant additionally requires K % 64 == 0 (kernels/nvfp4_gemv.cu:905).
int launch_nvfp4_gemv_v7(const void* weight_packed, const void* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream) {
    if (K % 64 != 0) return NVFP4_ERR_SHAPE;
    return nvfp4::gemv_dispatch(weight_packed, weight_scales, activation, nullptr, output, M, K,
                                stream, 1, "launch_nvfp4_gemv_v7");
}

int launch_nvfp4_gemv2(const void* weight_packed, const void* weight_scales, const void* act0,
                       const void* act1, void* output, int M, int K, void* stream) {
    return nvfp4::gemv_dispatch(weight_packed, weight_scales, act0, act1, output, M, K, stream, 2,
                                "launch_nvfp4_gemv2");
}

// Tuning hook (no counterpart in the reference): warps per CTA (0 = auto, 2/4/8), resident CTAs
// per SM used to size the grid (0 = occupancy calculator), force_generic != 0 routes every call
// to the non-tensor-core kernel.  Returns 0, or -2 for an unsupported value.
int nvfp4_b200_gemv_config(int warps, int ctas_per_sm, int force_generic) {
    if (!(warps == 0 || warps == 2 || warps == 4 || warps == 8) || ctas_per_sm < 0)
        return NVFP4_ERR_SHAPE;
    nvfp4::g_cfg.warps = warps;
    nvfp4::g_cfg.ctas_per_sm = ctas_per_sm;
    nvfp4::g_cfg.force_generic = force_generic;
    return NVFP4_OK;
}

}  // extern "C"

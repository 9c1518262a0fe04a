// Batch-1 NVFP4 GEMV for sm_100a with the weights streamed through a shared-memory ring by bulk
// asynchronous copies (cp.async.bulk, completion on mbarriers):  out[m] = sum_k W[m][k] * act[k].
//
// Replaces the reference's decode GEMV (kernels/nvfp4_gemv.cu:499-574 v8 kernel, launchers
// :837-977) for the shapes it takes; gemv.cu keeps the register-streaming kernel for the rest
// (two activations, K % 256 != 0, weaker alignment).
//
// Why a ring: a decode step is a chain of ~400 dependent launches of 5-50 MB each, so what counts
// is how early a kernel's weight bytes are in flight and how little of the machine idles between
// kernels.  Weights never depend on the previous kernel, only the activation does.  So:
//   * one CTA per SM and kernel, at most half of an SM's shared memory and registers: the CTAs of
//     the NEXT kernel in the stream (programmatic dependent launch) become resident beside the
//     running ones;
//   * a producer warp fills the ring (up to ~90 KB per SM) with bulk copies BEFORE it waits for
//     the previous kernel; bytes in flight no longer depend on resident warps x registers;
//   * the consumer warps wait for the previous kernel, stage the activation in shared memory
//     (optionally RMS-normalised), and then drain the ring: the memory pipe stays busy across
//     the kernel boundary.
//
// Work split: CTA b owns the contiguous rows [b M / G, (b+1) M / G) (G CTAs), not whole 16-row
// tiles, so every SM streams the same number of bytes whatever M is (5120 rows on 148 SMs: 34 or
// 35 rows each).  Rows are processed in tiles of up to 16 (a partial last tile only copies its
// own rows); a tile is cut along K into chunks of KC weights = one ring stage: 16 row segments of
// KC/2 packed bytes followed by 16 segments of KC/16 scale bytes (one contiguous copy each when a
// chunk covers whole rows, else one copy per row segment issued by the producer warp's lanes).
//
// Arithmetic (same as gemv_mma_kernel): nibbles -> fp16 with cvt.rn.f16x2.e2m1x2 (exact);
// mma.sync.m16n8k16 with the weights as A; column n of B holds the activation of ONE 64-wide K
// sub-chunk in the k-slots of the lanes that hold that sub-chunk's weights, so an accumulator
// column is the exact-product fp32 sum of one 16-weight scale block of one row, which is then
// multiplied by 2^(scale byte - 127) and added to the row's fp32 sum.
// Shared-memory reads are conflict-free without padding: rows are a multiple of 128 bytes apart,
// so lanes of odd rows read the two 16-byte halves of their 32-byte piece in the opposite order,
// and B columns 4..7 carry the activation in that order for them.
//
// Every mbarrier wait is bounded; a wait that runs out records itself in a status word
// (nvfp4_gemv_status), the CTA stops waiting and still runs to its end.
#include <cstdio>

#include "common.cuh"
#include "ptx.cuh"
#include "gemv_stream.cuh"

namespace nvfp4 {

constexpr int GS_MAX_STAGES = 8;
constexpr uint32_t GS_SPIN_LIMIT = 1u << 21;

__device__ unsigned int g_gemv_status = 0;   // 0 ok; else 1 + id of the wait that ran out

__device__ __forceinline__ void gs_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void gs_pdl_wait() {
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
}
__device__ __forceinline__ uint64_t gs_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
    return p;
}
// global -> this CTA's shared memory, `bytes` (multiple of 16) landing on mbarrier `bar`
__device__ __forceinline__ void gs_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                            uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;\n" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void gs_lds128(uint32_t a, uint32_t (&r)[4]) {
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ uint2 gs_lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
// 16-byte shared-memory load executed only where pred != 0; other lanes keep their registers
__device__ __forceinline__ void gs_lds_x_pred(uint32_t a, uint32_t pred, uint32_t& r0, uint32_t& r1,
                                              uint32_t& r2, uint32_t& r3) {
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.u32 p, %4, 0;\n"
                 "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%5];\n"
                 "}\n"
                 : "+r"(r0), "+r"(r1), "+r"(r2), "+r"(r3)
                 : "r"(pred), "r"(a));
}
__device__ __forceinline__ void gs_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// byte q (0..3) of w as an E8M0 scale in fp32 (byte 0 -> +0, byte 255 -> +inf)
__device__ __forceinline__ float gs_scale_byte(uint32_t w, int q) {
    if (q == 3) return __uint_as_float((w >> 1) & 0x7F800000u);
    return __uint_as_float((w & (0xFFu << (8 * q))) * (1u << (23 - 8 * q)));
}
// the consumer warps' own barrier (the producer warp never joins it)
template <int CW>
__device__ __forceinline__ void gs_consumer_sync() {
    asm volatile("bar.sync 1, %0;\n" ::"n"(CW * 32) : "memory");
}

// Bounded wait on an mbarrier phase.  `abort_flag` lets the other warps of a CTA leave quickly
// once one of them has given up.
__device__ __forceinline__ bool gs_wait(uint32_t bar, uint32_t parity, int id,
                                        volatile int* abort_flag) {
    for (uint32_t i = 0; i < GS_SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    atomicExch(&g_gemv_status, 1u + (unsigned)id);
    *abort_flag = 1;
    return false;
}

// CW consumer warps + 1 producer warp.  PRO / EPI as in gemv.cu (GS_PRO_*, GS_EPI_*).
// LATE: request the second 16-byte half of a lane's weights only after the first half has been
// consumed (fewer live registers, one more shared-memory round trip per step).
template <int CW, int PRO, int EPI, bool LATE>
__global__ void __launch_bounds__((CW + 1) * 32, 2)
gemv_stream_kernel(const StreamArgs a) {
    extern __shared__ __align__(128) uint8_t gs_smem[];
    __shared__ __align__(8) uint64_t bar_full[GS_MAX_STAGES];
    __shared__ __align__(8) uint64_t bar_empty[GS_MAX_STAGES];
    __shared__ float red[GS_MAX_STAGES][CW][16];
    __shared__ int cnt[GS_MAX_STAGES];
    __shared__ float s_part[CW];
    __shared__ int s_abort;

    gs_pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = a.K, KC = a.KC, nst = a.nst;
    const uint32_t xs_addr = smem_u32(gs_smem);
    const uint32_t ring_addr = xs_addr + (((uint32_t)K * 2u + 127u) & ~127u);

    // rows of this CTA, tiles and chunks
    const long long units = a.M / a.gran;
    const int r0 = (int)(((long long)blockIdx.x * units) / gridDim.x) * a.gran;
    const int r1 = (int)(((long long)(blockIdx.x + 1) * units) / gridDim.x) * a.gran;
    const int nt = (r1 - r0 + 15) >> 4;
    const int nc = (K + KC - 1) / KC;
    const int total = nt * nc;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nst; s++) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), CW);
        }
        for (int s = 0; s < GS_MAX_STAGES; s++) cnt[s] = 0;
        s_abort = 0;
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == CW) {
        // ------------------------------------------------------------------ producer warp
        const size_t prow = (size_t)(K >> 1), srow = (size_t)(K >> 4);
        const uint64_t policy = gs_policy_evict_first();
        int tile = 0, chunk = 0, slot = 0;
        uint32_t round = 0;               // s / nst
        int issued = 0;
        for (int s = 0; s < total; s++) {
            // The first ring fill needs nothing from the previous kernel.  Before the first wait
            // on a consumer, join the dependency: the consumers sit in griddepcontrol.wait until
            // the previous kernel has finished, which may take arbitrarily long, and a spin with
            // a limit must not span that.
            if (s == nst) gs_pdl_wait();
            if (s >= nst &&
                !gs_wait(smem_u32(&bar_empty[slot]), (round - 1u) & 1u, 0, &s_abort))
                break;
            const int row0 = r0 + tile * 16;
            const int nrows = min(16, r1 - row0);
            const int k0 = chunk * KC;
            const int kc = min(KC, K - k0);
            const uint32_t pb = (uint32_t)kc >> 1, sb = (uint32_t)kc >> 4;
            const uint32_t st = ring_addr + (uint32_t)slot * (uint32_t)a.stage_bytes;
            const uint32_t bar = smem_u32(&bar_full[slot]);
            if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)nrows * (pb + sb));
            __syncwarp();
            if (kc == K) {      // whole rows: the tile is one contiguous slab in each array
                if (lane == 0)
                    gs_bulk_g2s(st, a.packed + (size_t)row0 * prow, (uint32_t)nrows * pb, bar, policy);
                if (lane == 1)
                    gs_bulk_g2s(st + 16u * pb, a.scales + (size_t)row0 * srow, (uint32_t)nrows * sb,
                                bar, policy);
            } else {
                const int r = lane & 15;
                if (r < nrows) {
                    if (lane < 16)
                        gs_bulk_g2s(st + (uint32_t)r * pb,
                                    a.packed + (size_t)(row0 + r) * prow + (size_t)(k0 >> 1), pb, bar,
                                    policy);
                    else
                        gs_bulk_g2s(st + 16u * pb + (uint32_t)r * sb,
                                    a.scales + (size_t)(row0 + r) * srow + (size_t)(k0 >> 4), sb, bar,
                                    policy);
                }
            }
            issued = s + 1;
            if (++chunk == nc) { chunk = 0; tile++; }
            if (++slot == nst) { slot = 0; round++; }
        }
        // No copy may still be in flight into this CTA's shared memory when it exits: wait
        // (bounded) for the landing of the last copies issued into every slot.  In a normal run
        // the consumers have already seen all of them and these waits return at once.
        if (lane == 0) {
            for (int s = max(0, issued - nst); s < issued; s++)
                gs_wait(smem_u32(&bar_full[s % nst]), (uint32_t)(s / nst) & 1u, 3, &s_abort);
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int g = lane >> 2, t = lane & 3, p = g & 1;
    const uint32_t sup = ((g & 3) == t) ? 1u : 0u;   // this lane feeds column g of B
    const uint32_t ps = (uint32_t)g >> 2;            // ... which serves the rows of this parity
    constexpr int T = CW * 32;
    constexpr int NV = (CW >= 12) ? 2 : 3;           // 16-byte activation vectors per thread (RMSNorm)

    float4 wv[NV][2];
    if (PRO == GS_PRO_RMSNORM) {
        // the norm weights are constants: fetched while the previous kernel is still running
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = ((int)threadIdx.x + j * T) * 8;
            if (i < K) {
                wv[j][0] = __ldg(reinterpret_cast<const float4*>(a.norm_w1 + i));
                wv[j][1] = __ldg(reinterpret_cast<const float4*>(a.norm_w1 + i + 4));
            }
        }
    }
    gs_pdl_wait();
    const __half* act = a.act;
    asm volatile("" : "+l"(act));    // keep every activation read behind the wait

    if (PRO == GS_PRO_RMSNORM) {
        // x' = f16(f32(x) * rsqrt(mean(x^2) + eps) * w1): the arithmetic of rmsnorm_kernel
        uint4 xv[NV];
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = ((int)threadIdx.x + j * T) * 8;
            xv[j] = (i < K) ? *reinterpret_cast<const uint4*>(act + i) : make_uint4(0u, 0u, 0u, 0u);
        }
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const __half2* h = reinterpret_cast<const __half2*>(&xv[j]);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 f = __half22float2(h[e]);
                ss = fmaf(f.x, f.x, ss);
                ss = fmaf(f.y, f.y, ss);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) s_part[warp] = ss;
        gs_consumer_sync<CW>();
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < CW; w++) v += s_part[w];
        const float inv = rsqrtf(v / (float)K + a.eps);
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int i = ((int)threadIdx.x + j * T) * 8;
            if (i < K) {
                const __half2* h = reinterpret_cast<const __half2*>(&xv[j]);
                const float w[8] = {wv[j][0].x, wv[j][0].y, wv[j][0].z, wv[j][0].w,
                                    wv[j][1].x, wv[j][1].y, wv[j][1].z, wv[j][1].w};
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(h[e]);
                    oh[e] = __halves2half2(__float2half(f.x * inv * w[2 * e]),
                                           __float2half(f.y * inv * w[2 * e + 1]));
                }
                *reinterpret_cast<uint4*>(gs_smem + (size_t)i * 2) = o;
            }
        }
    } else {
        for (int i = (int)threadIdx.x * 8; i < K; i += T * 8)
            *reinterpret_cast<uint4*>(gs_smem + (size_t)i * 2) =
                *reinterpret_cast<const uint4*>(act + i);
    }
    gs_consumer_sync<CW>();

    float acc_a = 0.0f, acc_b = 0.0f;
    uint32_t x[8];
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = 0u;

    int tile = 0, chunk = 0, slot = 0;
    uint32_t phase = 0;
    int j0 = warp;                  // this warp's first step inside the current stage
    for (int s = 0; s < total; s++) {
        const int k0 = chunk * KC;
        const int kc = min(KC, K - k0);
        const int spc = kc >> 8;                               // 256-weight steps in this stage
        const uint32_t pb = (uint32_t)kc >> 1, sb = (uint32_t)kc >> 4;
        if (!gs_wait(smem_u32(&bar_full[slot]), phase, 1, &s_abort)) break;
        const uint32_t st = ring_addr + (uint32_t)slot * (uint32_t)a.stage_bytes;
        for (int j = j0; j < spc; j += CW) {
            // lane (g,t): 32 packed bytes (4 scale blocks) of row g and of row g+8; rows of odd g
            // take the two 16-byte halves in the opposite order
            const uint32_t wa = st + (uint32_t)g * pb + (uint32_t)j * 128u + (uint32_t)t * 32u;
            const uint32_t wb = wa + 8u * pb;
            uint32_t A[2][4], B[2][4];
            gs_lds128(wa + (uint32_t)p * 16u, A[0]);
            gs_lds128(wb + (uint32_t)p * 16u, B[0]);
            if (!LATE) {
                gs_lds128(wa + (uint32_t)(p ^ 1) * 16u, A[1]);
                gs_lds128(wb + (uint32_t)(p ^ 1) * 16u, B[1]);
            }
            const uint32_t sa_addr = st + 16u * pb + (uint32_t)g * sb + (uint32_t)j * 16u +
                                     (uint32_t)(t & 1) * 8u;
            uint2 sa = gs_lds64(sa_addr), sbv = gs_lds64(sa_addr + 8u * sb);
            if (p) {    // blocks 2,3 come first for odd rows
                sa.x = __byte_perm(sa.x, 0u, 0x1032);
                sa.y = __byte_perm(sa.y, 0u, 0x1032);
                sbv.x = __byte_perm(sbv.x, 0u, 0x1032);
                sbv.y = __byte_perm(sbv.y, 0u, 0x1032);
            }
            const uint32_t xa = xs_addr + (uint32_t)(k0 + j * 256 + t * 64) * 2u;
#pragma unroll
            for (int ph = 0; ph < 2; ph++) {
                if (LATE && ph == 1) {
                    gs_lds128(wa + (uint32_t)(p ^ 1) * 16u, A[1]);
                    gs_lds128(wb + (uint32_t)(p ^ 1) * 16u, B[1]);
                }
                const uint32_t xo = xa + (((uint32_t)ph ^ ps) * 64u);
#pragma unroll
                for (int bq = 0; bq < 2; bq++) {
                    gs_lds_x_pred(xo + bq * 32, sup, x[0], x[1], x[2], x[3]);
                    gs_lds_x_pred(xo + bq * 32 + 16, sup, x[4], x[5], x[6], x[7]);
                    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                        e2m1x8_to_half2x4(A[ph][2 * bq + h], a0, a1, a2, a3);
                        e2m1x8_to_half2x4(B[ph][2 * bq + h], b0, b1, b2, b3);
                        gs_mma(c, a0, b0, a1, b1, x[4 * h + 0], x[4 * h + 1]);
                        gs_mma(c, a2, b2, a3, b3, x[4 * h + 2], x[4 * h + 3]);
                    }
                    const int q = 2 * ph + bq;
                    acc_a = fmaf(c[0], gs_scale_byte(sa.x, q), acc_a);
                    acc_a = fmaf(c[1], gs_scale_byte(sa.y, q), acc_a);
                    acc_b = fmaf(c[2], gs_scale_byte(sbv.x, q), acc_b);
                    acc_b = fmaf(c[3], gs_scale_byte(sbv.y, q), acc_b);
                }
            }
        }
        j0 = (j0 - spc) % CW;
        if (j0 < 0) j0 += CW;

        if (chunk == nc - 1) {
            // ---- end of a row tile: combine the warps' partial sums; the warp that arrives last
            // adds them in warp order and writes the tile's outputs ----
            const int rs = tile & (GS_MAX_STAGES - 1);
            // columns 2t, 2t+1 of lane (g,t) belong to rows of parity t >> 1: lanes with
            // (t >> 1) == p hold this row's sums, the pair t = 2p, 2p+1
            acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
            acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
            if (t == 2 * p) {
                red[rs][warp][g] = acc_a;
                red[rs][warp][g + 8] = acc_b;
            }
            acc_a = 0.0f;
            acc_b = 0.0f;
            __syncwarp();
            int old = 0;
            if (lane == 0) {
                __threadfence_block();
                old = atomicAdd(&cnt[rs], 1);
            }
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == CW - 1) {
                __threadfence_block();
                float v = 0.0f;
                if (lane < 16) {
#pragma unroll
                    for (int w = 0; w < CW; w++) v += red[rs][w][lane];
                }
                const int row = r0 + tile * 16 + lane;
                if (EPI == GS_EPI_SILU_MUL) {
                    const float u = __shfl_down_sync(0xffffffffu, v, 8);
                    if (lane < 8 && row + 8 < r1) {
                        const float gf = round_f16(v), uf = round_f16(u);
                        const float sl = round_f16(gf / (1.0f + expf(-gf)));
                        a.out[(r0 >> 1) + tile * 8 + lane] = __float2half(sl * uf);
                    }
                } else if (lane < 16 && row < r1) {
                    if (EPI == GS_EPI_RESIDUAL)
                        a.out[row] = __float2half(__half2float(a.residual[row]) + round_f16(v));
                    else
                        a.out[row] = __float2half(v);
                }
                __syncwarp();
                if (lane == 0) cnt[rs] = 0;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_empty[slot]));
        if (++chunk == nc) { chunk = 0; tile++; }
        if (++slot == nst) { slot = 0; phase ^= 1u; }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static StreamConfig g_scfg;

StreamConfig& stream_config() { return g_scfg; }

static int device_sms() {
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

bool plan_stream(int M, int K, int prologue, int epilogue, StreamPlan* out) {
    if (g_scfg.disable) return false;
    if (K % 256 != 0 || M <= 0) return false;
    const int cw = g_scfg.warps ? g_scfg.warps : 16;
    const int nv = (cw >= 12) ? 2 : 3;
    if (prologue == GS_PRO_RMSNORM && K > nv * 8 * cw * 32) return false;
    const int budget = (g_scfg.smem_kb ? g_scfg.smem_kb : 100) * 1024;
    const int xs = (2 * K + 127) & ~127;
    const int ring = budget - xs;
    const int min_st = g_scfg.min_stages ? g_scfg.min_stages : 3;
    int kc_fit = ring / min_st / 9 / 256 * 256;
    int kc_tgt = (g_scfg.stage_kb ? g_scfg.stage_kb : 24) * 1024 / 9 / 256 * 256;
    int kcmax = kc_fit < kc_tgt ? kc_fit : kc_tgt;
    if (kcmax > K) kcmax = K;
    if (kcmax < 256) return false;
    const int nc = (K + kcmax - 1) / kcmax;
    const int KC = ((K + nc - 1) / nc + 255) / 256 * 256;
    const int stage = 9 * KC;
    int nst = ring / stage;
    if (nst > GS_MAX_STAGES) nst = GS_MAX_STAGES;
    if (nst < 2) return false;
    const int gran = (epilogue == GS_EPI_SILU_MUL) ? 16 : 1;
    if (M % gran != 0) return false;
    const long long units = M / gran;
    int grid = device_sms() * (g_scfg.ctas_per_sm ? g_scfg.ctas_per_sm : 1);
    if (grid > units) grid = (int)units;
    out->warps = cw;
    out->KC = KC;
    out->nst = nst;
    out->stage_bytes = stage;
    out->gran = gran;
    out->grid = grid;
    out->smem = xs + nst * stage;
    // 16 consumer warps have 56 registers each when two CTAs share an SM: the late second-half
    // load keeps that variant free of spills
    out->late = (g_scfg.late == 0) ? (cw >= 16 ? 1 : 0) : (g_scfg.late > 0 ? 1 : 0);
    return true;
}

template <int CW, int PRO, int EPI, bool LATE>
static cudaError_t launch_stream_t(const StreamArgs& a, const StreamPlan& pl, cudaStream_t st,
                                   bool pdl) {
    // the opt-in to large dynamic shared memory is per device
    static int set_for[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && set_for[dev] < pl.smem) {
        const cudaError_t e =
            cudaFuncSetAttribute(gemv_stream_kernel<CW, PRO, EPI, LATE>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
        if (e != cudaSuccess) return e;
        // ask for the largest shared-memory carve-out so that two CTAs (this kernel's and the
        // next kernel's) fit on an SM side by side
        cudaFuncSetAttribute(gemv_stream_kernel<CW, PRO, EPI, LATE>,
                             cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared);
        set_for[dev] = 110 * 1024;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.grid);
    cfg.blockDim = dim3((CW + 1) * 32);
    cfg.dynamicSmemBytes = (size_t)pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<CW, PRO, EPI, LATE>, a);
}

template <int CW, bool LATE>
static cudaError_t launch_stream_cw(const StreamArgs& a, const StreamPlan& pl, int pro, int epi,
                                    cudaStream_t st, bool pdl) {
#define GS_CASE(P, E) return launch_stream_t<CW, P, E, LATE>(a, pl, st, pdl)
    if (pro == GS_PRO_NONE) {
        if (epi == GS_EPI_STORE) GS_CASE(GS_PRO_NONE, GS_EPI_STORE);
        if (epi == GS_EPI_RESIDUAL) GS_CASE(GS_PRO_NONE, GS_EPI_RESIDUAL);
        GS_CASE(GS_PRO_NONE, GS_EPI_SILU_MUL);
    }
    if (epi == GS_EPI_STORE) GS_CASE(GS_PRO_RMSNORM, GS_EPI_STORE);
    if (epi == GS_EPI_RESIDUAL) GS_CASE(GS_PRO_RMSNORM, GS_EPI_RESIDUAL);
    GS_CASE(GS_PRO_RMSNORM, GS_EPI_SILU_MUL);
#undef GS_CASE
}

cudaError_t launch_stream(const void* packed, const void* scales, const void* act, void* out, int M,
                          int K, int pro, const void* norm_w1, float eps, int epi,
                          const void* residual, const StreamPlan& pl, cudaStream_t st, bool pdl) {
    StreamArgs a;
    a.packed = (const uint8_t*)packed;
    a.scales = (const uint8_t*)scales;
    a.act = (const __half*)act;
    a.out = (__half*)out;
    a.norm_w1 = (const float*)norm_w1;
    a.residual = (const __half*)residual;
    a.eps = eps;
    a.M = M;
    a.K = K;
    a.KC = pl.KC;
    a.nst = pl.nst;
    a.stage_bytes = pl.stage_bytes;
    a.gran = pl.gran;
    const bool late = pl.late != 0;
    switch (pl.warps) {
        case 8: return late ? launch_stream_cw<8, true>(a, pl, pro, epi, st, pdl)
                            : launch_stream_cw<8, false>(a, pl, pro, epi, st, pdl);
        case 12: return late ? launch_stream_cw<12, true>(a, pl, pro, epi, st, pdl)
                             : launch_stream_cw<12, false>(a, pl, pro, epi, st, pdl);
        default: return late ? launch_stream_cw<16, true>(a, pl, pro, epi, st, pdl)
                             : launch_stream_cw<16, false>(a, pl, pro, epi, st, pdl);
    }
}

}  // namespace nvfp4

extern "C" {

// 0 if no bounded wait inside the ring GEMV has run out since the library was loaded (or since
// the last call with reset != 0); otherwise 1 + the id of the wait (0 producer waiting for a free
// stage, 1 consumer waiting for a stage's bytes, 3 final drain).  Synchronises the device.
int nvfp4_gemv_status(int reset) {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, nvfp4::g_gemv_status, sizeof(v)) != cudaSuccess) return -1;
    if (reset) {
        const unsigned int z = 0;
        cudaMemcpyToSymbol(nvfp4::g_gemv_status, &z, sizeof(z));
    }
    return (int)v;
}

// Tuning hook of the ring GEMV (no counterpart in the reference): consumer warps per CTA (0 = 16;
// 8, 12, 16), shared-memory budget per CTA in KB (0 = 100), target stage size in KB (0 = 24),
// minimum ring stages (0 = 3), CTAs per SM used to size the grid (0 = 1), late: 0 = automatic,
// 1 / -1 = force / forbid the late second-half load, disable != 0 routes every GEMV to the
// register-streaming kernel.  Process-wide, not thread-safe.  0 or -2.
int nvfp4_b200_gemv_stream_config(int warps, int smem_kb, int stage_kb, int min_stages,
                                  int ctas_per_sm, int late, int disable) {
    if (!(warps == 0 || warps == 8 || warps == 12 || warps == 16)) return NVFP4_ERR_SHAPE;
    if (smem_kb < 0 || smem_kb > 108 || stage_kb < 0 || min_stages < 0 || min_stages > 8 ||
        ctas_per_sm < 0 || ctas_per_sm > 2)
        return NVFP4_ERR_SHAPE;
    nvfp4::StreamConfig& c = nvfp4::stream_config();
    c.warps = warps;
    c.smem_kb = smem_kb;
    c.stage_kb = stage_kb;
    c.min_stages = min_stages;
    c.ctas_per_sm = ctas_per_sm;
    c.late = late;
    c.disable = disable;
    return NVFP4_OK;
}

}  // extern "C"

// Batch-1 NVFP4 GEMV for sm_100a with the weights streamed through a shared-memory ring by TMA
// tensor copies (cp.async.bulk.tensor.2d, completion on mbarriers):
//     out[m] = sum_k W[m][k] * act[k].
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
//   * a producer warp fills the ring (up to ~90 KB per SM) BEFORE it waits for the previous
//     kernel; bytes in flight no longer depend on resident warps x registers;
//   * the consumer warps wait for the previous kernel, stage the activation in shared memory
//     (optionally RMS-normalised), and then drain the ring.
//
// Work split: the rows are dealt to the CTAs in units of RB rows (4 or 16), CTA b owning the
// contiguous units [b U / G, (b+1) U / G), so every SM streams nearly the same number of bytes
// whatever M is (5120 rows on 148 SMs: 32 or 36 rows each).  Rows are processed in tiles of up to
// 16; a tile is cut along K into chunks of KC weights = one ring stage: 16 row segments of KC/2
// packed bytes, then 16 segments of KC/16 scale bytes, fetched as boxes of RB rows x KC by two
// tensor maps over the raw [M][K/2] and [M][K/16] arrays (elements outside the arrays read as
// zero, so ragged K chunks and a ragged last row box need no special case).  Measured on B200:
// a plain cp.async.bulk per row segment costs ~45 ns of issue time each whatever its size, which
// caps a ring fed that way at ~16 GB/s per SM; a tensor copy moves a whole box per instruction.
//
// Arithmetic (same as gemv_mma_kernel): nibbles -> fp16 with cvt.rn.f16x2.e2m1x2 (exact, one
// machine instruction per byte); mma.sync.m16n8k16 with the weights as A; column n of B holds the
// activation of ONE 64-wide K sub-chunk in the k-slots of the lanes that hold that sub-chunk's
// weights, so an accumulator column is the exact-product fp32 sum of one 16-weight scale block of
// one row, which is then multiplied by 2^(scale byte - 127) and added to the row's fp32 sum.
// Shared-memory reads are conflict-free without padding the weights: rows are a multiple of 128
// bytes apart, so lanes of odd rows read the two 16-byte halves of their 32-byte piece in the
// opposite order, and B columns 4..7 carry the activation in that order for them.  The
// activation is stored with 16 bytes of padding per 128 so that the eight lanes that feed B read
// eight different bank groups; the other lanes read a zero slot.
//
// Every mbarrier wait is bounded; a wait that runs out records itself in a status word
// (nvfp4_gemv_status), the CTA stops waiting and still runs to its end.
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"
#include "gemv_stream.cuh"

namespace nvfp4 {

constexpr int GS_MAX_DEPTH = 4;      // stages of a warp's private ring
constexpr int GS_RED_DEPTH = 4;     // row tiles whose partial sums may be outstanding at once
constexpr int GS_MAX_CHUNKS = 24;   // K chunks per row tile
constexpr uint32_t GS_SPIN_LIMIT = 1u << 20;   // tries of up to 4 us each

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
// one box of a 2-D tensor map -> this CTA's shared memory, landing on mbarrier `bar`
__device__ __forceinline__ void gs_tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                          uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;\n" ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar),
        "l"(policy)
        : "memory");
}
// fp16 x fp16 -> fp32 tensor-core product; the accumulator starts at zero (ZERO) or continues
template <bool ZERO>
__device__ __forceinline__ void gs_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
    if (ZERO) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%10,%10,%10,%10};\n"
            : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}
// byte q (0..3) of w as an E8M0 scale in fp32 (byte 0 -> +0, byte 255 -> +inf)
__device__ __forceinline__ float gs_scale_byte(uint32_t w, int q) {
    if (q == 3) return __uint_as_float((w >> 1) & 0x7F800000u);
    return __uint_as_float((w & (0xFFu << (8 * q))) * (1u << (23 - 8 * q)));
}
// Bounded wait on an mbarrier phase.  `abort_flag` lets the other warps of a CTA leave quickly
// once one of them has given up.
__device__ __forceinline__ bool gs_wait(uint32_t bar, uint32_t parity, int id,
                                        volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < GS_SPIN_LIMIT; i++) {
        if (mbar_try_wait_hint(bar, parity, 4000u)) return true;    // parked, not spinning
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    atomicExch(&g_gemv_status, 1u + (unsigned)id);
    *abort_flag = 1;
    return false;
}

// byte offset of activation element k in the padded shared-memory copy (16 bytes after every 128)
__device__ __forceinline__ uint32_t gs_x_off(uint32_t k) { return k * 2u + (k >> 6) * 16u; }

// CW warps, each with a private ring of D stages that it fills itself.  PRO / EPI: GS_PRO_*,
// GS_EPI_*.
//
// Work units: (row tile, K chunk) pairs in row-major order; unit u belongs to warp u % CW, which
// processes ALL of its KC/256 steps without meeting another warp, and whose lane 0 then refills
// the stage with the warp's unit D places ahead: no producer warp, no "stage free" barrier, no
// warp ever waits for another one's progress.  (Two earlier arrangements measured slower: every
// stage shared by all warps, one step each, cost 311 instructions and 160 clocks per step against
// 185 and 77 for the bare step, because the barrier visit cost as much as the step; a producer
// warp feeding per-warp stages in unit order let the slowest warp hold up the refills of all.)
// The nc units of a tile leave their 16 partial sums in shared memory; the unit that arrives last
// adds them in chunk order (deterministic) and writes the outputs.
template <int CW, int PRO, int EPI>
__global__ void __launch_bounds__(CW * 32, 1)
gemv_stream_kernel(const __grid_constant__ CUtensorMap map_p16,
                   const __grid_constant__ CUtensorMap map_s16,
                   const __grid_constant__ CUtensorMap map_p4,
                   const __grid_constant__ CUtensorMap map_s4, const StreamArgs a) {
    extern __shared__ __align__(128) uint8_t gs_smem[];
    __shared__ __align__(8) uint64_t bar_full[CW][GS_MAX_DEPTH];
    __shared__ float red[GS_RED_DEPTH][GS_MAX_CHUNKS][16];
    __shared__ int cnt[GS_RED_DEPTH];
    __shared__ int gen[GS_RED_DEPTH];      // how many tiles have finished with each `red` slot
    __shared__ float s_part[CW];
    __shared__ int s_abort;

    gs_pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = a.K, KC = a.KC, D = a.nst, RB = a.rb;
    // shared memory: 128 zero bytes, the padded activation, the rings
    uint8_t* const xs = gs_smem + 128;
    uint8_t* const ring = gs_smem + a.ring_off + (size_t)warp * (size_t)D * (size_t)a.stage_bytes;

    // rows of this CTA (units of RB rows), tiles and chunks
    const long long units = (a.M + RB - 1) / RB;
    const int r0 = (int)(((long long)blockIdx.x * units) / gridDim.x) * RB;
    const int r1 = min(a.M, (int)(((long long)(blockIdx.x + 1) * units) / gridDim.x) * RB);
    const int nt = (r1 - r0 + 15) >> 4;
    const int nc = (K + KC - 1) / KC;
    const int total = nt * nc;
    const int n_my = (warp < total) ? (total - warp + CW - 1) / CW : 0;   // this warp's units
    const uint32_t pb = (uint32_t)KC >> 1, sb = (uint32_t)KC >> 4;   // bytes per row and stage

    if (threadIdx.x == 0) {
        for (int w = 0; w < CW; w++)
            for (int d = 0; d < D; d++) mbar_init(smem_u32(&bar_full[w][d]), 1);
        for (int s = 0; s < GS_RED_DEPTH; s++) { cnt[s] = 0; gen[s] = 0; }
        s_abort = 0;
        fence_barrier_init();
    }
    if (threadIdx.x < 32) reinterpret_cast<uint32_t*>(gs_smem)[threadIdx.x] = 0u;   // zero slots
    __syncthreads();

    // lane 0: fetch this warp's unit (tile, chunk) into stage d of its ring
    const uint64_t policy = gs_policy_evict_first();
    auto issue = [&](int tile, int chunk, int d) {
        const int row0 = r0 + tile * 16;
        const int nrows = min(16, r1 - row0);
        const uint32_t st = smem_u32(ring) + (uint32_t)d * (uint32_t)a.stage_bytes;
        const uint32_t bar = smem_u32(&bar_full[warp][d]);
        if (a.probe & 2) {       // attribution probe: no weight traffic at all
            mbar_arrive(bar);
            return;
        }
        const int c0 = (chunk * KC) >> 4;   // u64 elements of packed = bytes of scales
        if (nrows == 16) {
            mbar_arrive_expect_tx(bar, 16u * (pb + sb));
            gs_tma_2d(st, &map_p16, c0, row0, bar, policy);
            gs_tma_2d(st + 16u * pb, &map_s16, c0, row0, bar, policy);
        } else {             // ragged last tile of the CTA: boxes of four rows
            const int boxes = (nrows + 3) >> 2;
            mbar_arrive_expect_tx(bar, (uint32_t)(boxes * 4) * (pb + sb));
            for (int b = 0; b < boxes; b++) {
                gs_tma_2d(st + (uint32_t)(b * 4) * pb, &map_p4, c0, row0 + b * 4, bar, policy);
                gs_tma_2d(st + 16u * pb + (uint32_t)(b * 4) * sb, &map_s4, c0, row0 + b * 4, bar,
                          policy);
            }
        }
    };
    // (tile, chunk) of the unit the refill pointer is at; it runs D units ahead of the compute
    int ftile = warp / nc, fchunk = warp % nc;
    auto advance = [&](int& tile, int& chunk) {
        chunk += CW;
        while (chunk >= nc) { chunk -= nc; tile++; }
    };
    // The first ring fill needs nothing from the previous kernel: weights are constants.
    {
        const int pre = min(D, n_my);
        for (int i = 0; i < pre; i++) {
            if (lane == 0) issue(ftile, fchunk, i);
            advance(ftile, fchunk);
        }
    }

    const int g = lane >> 2, t = lane & 3, p = g & 1;
    const bool sup = ((g & 3) == t);                 // this lane feeds column g of B
    const uint32_t ps = (uint32_t)g >> 2;            // ... which serves the rows of this parity
    constexpr int T = CW * 32;
    constexpr int NV = (6144 + 8 * T - 1) / (8 * T);  // 16-byte activation vectors per thread (RMSNorm)

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
        __syncthreads();
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
                *reinterpret_cast<uint4*>(xs + gs_x_off((uint32_t)i)) = o;
            }
        }
    } else {
        for (int i = (int)threadIdx.x * 8; i < K; i += T * 8)
            *reinterpret_cast<uint4*>(xs + gs_x_off((uint32_t)i)) =
                *reinterpret_cast<const uint4*>(act + i);
    }
    __syncthreads();

    // Lanes that do not feed B read 16 zero bytes instead (a slot per quarter-warp).
    const uint8_t* const zslot = gs_smem + (((lane >> 3) * 2 + 2) & 7) * 16;
    const uint32_t wlane = (uint32_t)g * pb + (uint32_t)t * 32u;
    const uint32_t slane = 16u * pb + (uint32_t)g * sb + (uint32_t)(t & 1) * 8u;

    int tile = warp / nc, chunk = warp % nc, d = 0, done_units = 0;
    uint32_t phase = 0;
    for (int i = 0; i < n_my; i++) {
        const int k0 = chunk * KC;
        const int spc = min(KC, K - k0) >> 8;                  // valid 256-weight steps in this unit
        if (!gs_wait(smem_u32(&bar_full[warp][d]), phase, 1, &s_abort)) break;
        const uint8_t* const st = ring + (size_t)d * (size_t)a.stage_bytes;
        const uint8_t* wa = st + wlane;
        const uint8_t* sp = st + slane;
        const uint8_t* xa = xs + gs_x_off((uint32_t)(k0 + t * 64));
        float acc_a = 0.0f, acc_b = 0.0f;
        for (int j = (a.probe & 1) ? spc : 0; j < spc; j++) {   // probe bit 0: no arithmetic
            // lane (g,t): 32 packed bytes (4 scale blocks) of row g and of row g+8; rows of odd g
            // take the two 16-byte halves in the opposite order
            const uint8_t* const wb = wa + 8u * pb;
            uint4 A[2], B[2];
            A[0] = *reinterpret_cast<const uint4*>(wa + p * 16);
            B[0] = *reinterpret_cast<const uint4*>(wb + p * 16);
            A[1] = *reinterpret_cast<const uint4*>(wa + (p ^ 1) * 16);
            B[1] = *reinterpret_cast<const uint4*>(wb + (p ^ 1) * 16);
            uint2 sa = *reinterpret_cast<const uint2*>(sp);
            uint2 sbv = *reinterpret_cast<const uint2*>(sp + 8u * sb);
            if (p) {    // blocks 2,3 come first for odd rows
                sa.x = __byte_perm(sa.x, 0u, 0x1032);
                sa.y = __byte_perm(sa.y, 0u, 0x1032);
                sbv.x = __byte_perm(sbv.x, 0u, 0x1032);
                sbv.y = __byte_perm(sbv.y, 0u, 0x1032);
            }
#pragma unroll
            for (int ph = 0; ph < 2; ph++) {
                const uint32_t aw[4] = {A[ph].x, A[ph].y, A[ph].z, A[ph].w};
                const uint32_t bw[4] = {B[ph].x, B[ph].y, B[ph].z, B[ph].w};
                const uint8_t* const xo = xa + (((uint32_t)ph ^ ps) * 64u);
#pragma unroll
                for (int bq = 0; bq < 2; bq++) {
                    const uint4 x0 = *reinterpret_cast<const uint4*>(sup ? xo + bq * 32 : zslot);
                    const uint4 x1 = *reinterpret_cast<const uint4*>(sup ? xo + bq * 32 + 16 : zslot);
                    const uint32_t x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                    float c[4];
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                        e2m1x8_to_half2x4(aw[2 * bq + h], a0, a1, a2, a3);
                        e2m1x8_to_half2x4(bw[2 * bq + h], b0, b1, b2, b3);
                        if (h == 0) gs_mma<true>(c, a0, b0, a1, b1, x[0], x[1]);
                        else gs_mma<false>(c, a0, b0, a1, b1, x[4], x[5]);
                        gs_mma<false>(c, a2, b2, a3, b3, x[4 * h + 2], x[4 * h + 3]);
                    }
                    const int q = 2 * ph + bq;
                    acc_a = fmaf(c[0], gs_scale_byte(sa.x, q), acc_a);
                    acc_a = fmaf(c[1], gs_scale_byte(sa.y, q), acc_a);
                    acc_b = fmaf(c[2], gs_scale_byte(sbv.x, q), acc_b);
                    acc_b = fmaf(c[3], gs_scale_byte(sbv.y, q), acc_b);
                }
            }
            wa += 128;
            sp += 16;
            xa += 4 * 144;       // 256 activations and their padding
        }
        // Every lane has used the stage's bytes (their consumers have issued): refill it with
        // the unit D places ahead.  The fence orders this warp's reads of the stage before the
        // copy engine's writes to it.
        __syncwarp();
        if (i + D < n_my) {
            if (lane == 0) {
                fence_proxy_async_smem();
                issue(ftile, fchunk, d);
            }
            advance(ftile, fchunk);
        }

        // ---- this unit's 16 partial row sums.  Columns 2t, 2t+1 of lane (g,t) belong to rows of
        // parity t >> 1: lanes with (t >> 1) == p hold this row's sums, the pair t = 2p, 2p+1.
        acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
        acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
        float v;        // lanes 0..15: the sum of row `lane` of the tile (valid in the finisher)
        bool finisher = true;
        if (nc == 1) {
            // one unit per tile: bring row r's sum to lane r (row g sits in lane 4g + 2p, row
            // g + 8 in the same lane's acc_b)
            const int src = 4 * (lane & 7) + 2 * (lane & 1);
            const float va = __shfl_sync(0xffffffffu, acc_a, src);
            const float vb = __shfl_sync(0xffffffffu, acc_b, src);
            v = (lane < 8) ? va : vb;
        } else {
            const int rs = tile & (GS_RED_DEPTH - 1);
            // The warps run independently, so one may be many tiles ahead of another: a `red`
            // slot is written only once the tile that used it before (GS_RED_DEPTH tiles back)
            // has been summed.  Bounded like every other wait here.
            {
                const int want = tile / GS_RED_DEPTH;
                uint32_t spins = 0;
                while (*reinterpret_cast<volatile int*>(&gen[rs]) != want) {
                    if (++spins > (1u << 24) || s_abort) {
                        atomicExch(&g_gemv_status, 5u);
                        s_abort = 1;
                        break;
                    }
                }
            }
            if (t == 2 * p) {
                red[rs][chunk][g] = acc_a;
                red[rs][chunk][g + 8] = acc_b;
            }
            __syncwarp();
            int old = 0;
            if (lane == 0) {
                __threadfence_block();
                old = atomicAdd(&cnt[rs], 1);
            }
            old = __shfl_sync(0xffffffffu, old, 0);
            finisher = (old == nc - 1);
            v = 0.0f;
            if (finisher) {     // the last unit of the tile to arrive adds them in chunk order
                __threadfence_block();
                if (lane < 16)
                    for (int c = 0; c < nc; c++) v += red[rs][c][lane];
                __syncwarp();
                if (lane == 0) {
                    cnt[rs] = 0;
                    __threadfence_block();
                    gen[rs] = tile / GS_RED_DEPTH + 1;
                }
            }
        }
        if (finisher) {
            const int row = r0 + tile * 16 + lane;
            if (EPI == GS_EPI_SILU_MUL) {
                const float up = __shfl_down_sync(0xffffffffu, v, 8);
                if (lane < 8 && row + 8 < r1) {
                    const float gf = round_f16(v), uf = round_f16(up);
                    const float sl = round_f16(gf / (1.0f + expf(-gf)));
                    a.out[(r0 >> 1) + tile * 8 + lane] = __float2half(sl * uf);
                }
            } else if (lane < 16 && row < r1) {
                if (EPI == GS_EPI_RESIDUAL)
                    a.out[row] = __float2half(__half2float(a.residual[row]) + round_f16(v));
                else
                    a.out[row] = __float2half(v);
            }
        }
        advance(tile, chunk);
        if (++d == D) { d = 0; phase ^= 1u; }
        done_units = i + 1;
    }
    // Only after a wait ran out: no copy may still be in flight into this CTA's shared memory
    // when it exits, so wait (bounded) for the units that were requested but not consumed.
    if (done_units < n_my) {
        const int issued = min(n_my, done_units + D);
        for (int k = done_units; k < issued; k++)
            gs_wait(smem_u32(&bar_full[warp][k % D]), (uint32_t)(k / D) & 1u, 3, &s_abort);
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static StreamConfig g_scfg;

StreamConfig& stream_config() { return g_scfg; }

static int device_sms() {
    static int cache[NVFP4_MAX_DEVICES] = {0};
    const int dev = current_device_index();
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

bool plan_stream(int M, int K, int prologue, int epilogue, StreamPlan* out) {
    if (!g_scfg.enable) return false;
    if (K % 256 != 0 || M <= 0) return false;
    if (encode_tiled_fn() == nullptr) return false;
    const int ctas = g_scfg.ctas_per_sm ? g_scfg.ctas_per_sm : 1;
    const int cw = g_scfg.warps ? g_scfg.warps : 8;
    const int nv = (6144 + 8 * cw * 32 - 1) / (8 * cw * 32);
    if (prologue == GS_PRO_RMSNORM && K > nv * 8 * cw * 32) return false;
    // static shared memory is about 13 KB; an SM has 227 KB for one CTA, 113 KB each for two
    const int budget = (g_scfg.smem_kb ? g_scfg.smem_kb : (ctas == 1 ? 208 : 98)) * 1024;
    const int xs = 128 + (((2 * K + (K / 64) * 16) + 127) & ~127);   // zero slots + padded activation
    const int ring = budget - xs;
    // K chunk of a work unit: a multiple of 512 weights (so that four scale rows are a multiple
    // of 128 bytes, the alignment a tensor copy's destination needs), at most 24 chunks per row
    int KC = (g_scfg.stage_kb ? g_scfg.stage_kb * 1024 / 9 : 1024) / 512 * 512;
    if (KC < 512) KC = 512;
    while ((K + KC - 1) / KC > GS_MAX_CHUNKS) KC += 512;
    if (KC > 4096) return false;             // a tensor-map box holds at most 256 elements per dim
    const int stage = 9 * KC;
    int depth = ring / (stage * cw);         // stages of each warp's private ring
    if (depth > GS_MAX_DEPTH) depth = GS_MAX_DEPTH;
    if (g_scfg.min_stages && depth > g_scfg.min_stages) depth = g_scfg.min_stages;   // tuning: cap
    if (depth < 2) return false;
    int grid = device_sms() * ctas;
    // rows are dealt to the CTAs in units of 4 (16 where the epilogue pairs gate and up rows)
    int rb = g_scfg.rows_per_box ? g_scfg.rows_per_box : 4;
    if (epilogue == GS_EPI_SILU_MUL) {
        if (M % 16 != 0) return false;
        rb = 16;
    }
    const long long units = (M + rb - 1) / rb;
    if (grid > units) grid = (int)units;
    out->warps = cw;
    out->KC = KC;
    out->nst = depth;
    out->stage_bytes = stage;
    out->rb = rb;
    out->grid = grid;
    out->ring_off = xs;
    out->smem = xs + cw * depth * stage;
    return true;
}

// Tensor maps of one weight matrix: packed bytes as [M][K/16] 8-byte elements, scale bytes as
// [M][K/16]; box = KC/16 elements x rb rows for both.  Encoding is pure host work (about a
// microsecond); a small cache keeps it off the path of callers that launch eagerly.
struct MapKey {
    const void* packed;
    const void* scales;
    int M, K, KC, rb;
    bool operator==(const MapKey& o) const {
        return packed == o.packed && scales == o.scales && M == o.M && K == o.K && KC == o.KC &&
               rb == o.rb;
    }
};
struct MapEntry {
    MapKey key;
    bool valid;
    CUtensorMap mp, ms;
};
static MapEntry g_maps[256];
static std::mutex g_maps_mutex;

static bool get_maps(const void* packed, const void* scales, int M, int K, int KC, int rb,
                     CUtensorMap* mp, CUtensorMap* ms) {
    const MapKey key = {packed, scales, M, K, KC, rb};
    const size_t h = ((((uintptr_t)packed >> 8) + (uintptr_t)rb) * 0x9E3779B97F4A7C15ull >> 40) & 255;
    {
        std::lock_guard<std::mutex> lock(g_maps_mutex);
        if (g_maps[h].valid && g_maps[h].key == key) {
            *mp = g_maps[h].mp;
            *ms = g_maps[h].ms;
            return true;
        }
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)(K / 16), (cuuint64_t)M};
    const cuuint32_t box[2] = {(cuuint32_t)(KC / 16), (cuuint32_t)rb};
    const cuuint32_t estr[2] = {1, 1};
    const cuuint64_t pstride[1] = {(cuuint64_t)(K / 2)};
    const cuuint64_t sstride[1] = {(cuuint64_t)(K / 16)};
    if (enc(mp, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(packed), dims, pstride, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (enc(ms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(scales), dims, sstride, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    g_maps[h].key = key;
    g_maps[h].mp = *mp;
    g_maps[h].ms = *ms;
    g_maps[h].valid = true;
    return true;
}

struct StreamMaps {
    CUtensorMap p16, s16, p4, s4;
};

template <int CW, int PRO, int EPI>
static cudaError_t launch_stream_t(const StreamMaps& m,
                                   const StreamArgs& a, const StreamPlan& pl, cudaStream_t st,
                                   bool pdl) {
    // the opt-in to large dynamic shared memory is per device
    static bool set_for[NVFP4_MAX_DEVICES] = {false};
    const int dev = current_device_index();
    if (!set_for[dev]) {
        const cudaError_t e =
            cudaFuncSetAttribute(gemv_stream_kernel<CW, PRO, EPI>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 212 * 1024);
        if (e != cudaSuccess) return e;
        // ask for the largest shared-memory carve-out
        cudaFuncSetAttribute(gemv_stream_kernel<CW, PRO, EPI>,
                             cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared);
        set_for[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.grid);
    cfg.blockDim = dim3(CW * 32);
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
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<CW, PRO, EPI>, m.p16, m.s16, m.p4, m.s4, a);
}

template <int CW>
static cudaError_t launch_stream_cw(const StreamMaps& m,
                                    const StreamArgs& a, const StreamPlan& pl, int pro, int epi,
                                    cudaStream_t st, bool pdl) {
#define GS_CASE(P, E) return launch_stream_t<CW, P, E>(m, a, pl, st, pdl)
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
    StreamMaps m;
    if (!get_maps(packed, scales, M, K, pl.KC, 16, &m.p16, &m.s16) ||
        !get_maps(packed, scales, M, K, pl.KC, 4, &m.p4, &m.s4))
        return cudaErrorInvalidValue;
    StreamArgs a;
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
    a.rb = pl.rb;
    a.ring_off = pl.ring_off;
    a.probe = g_scfg.probe;
    switch (pl.warps) {
        case 4: return launch_stream_cw<4>(m, a, pl, pro, epi, st, pdl);
        case 12: return launch_stream_cw<12>(m, a, pl, pro, epi, st, pdl);
        default: return launch_stream_cw<8>(m, a, pl, pro, epi, st, pdl);
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

// Switch and tuning hook of the ring GEMV (no counterpart in the reference).  flags bit 0 turns
// the ring kernel ON for the shapes it takes (it is off by default: on B200 the register-streaming
// kernel measured faster on every 27B layer shape); bits 4 and 5 are attribution probes that give
// WRONG results on purpose (bit 4: no arithmetic, a launch costs what its weight stream costs;
// bit 5: no weight copies, a launch costs what its arithmetic costs).  warps per CTA (0 = 8; 4, 8,
// 12), shared-memory budget per CTA in KB (0 = 208 with one CTA per SM, 98 with two), stage size
// in KB (0 = 9: 1024 weights of 16 rows), most stages per warp (0 = 4; 2..4), CTAs per SM used to
// size the grid (0 = 1), the unit in which rows are dealt to the CTAs (0 = 4; 4 or 16).
// Process-wide, not thread-safe.  0 or -2.
int nvfp4_b200_gemv_stream_config(int warps, int smem_kb, int stage_kb, int min_stages,
                                  int ctas_per_sm, int rows_per_box, int flags) {
    if (!(warps == 0 || warps == 4 || warps == 8 || warps == 12)) return NVFP4_ERR_SHAPE;
    if (smem_kb < 0 || smem_kb > 208 || stage_kb < 0 || min_stages < 0 || min_stages > 4 ||
        ctas_per_sm < 0 || ctas_per_sm > 2 ||
        !(rows_per_box == 0 || rows_per_box == 4 || rows_per_box == 16))
        return NVFP4_ERR_SHAPE;
    nvfp4::StreamConfig& c = nvfp4::stream_config();
    c.warps = warps;
    c.smem_kb = smem_kb;
    c.stage_kb = stage_kb;
    c.min_stages = min_stages;
    c.ctas_per_sm = ctas_per_sm;
    c.rows_per_box = rows_per_box;
    c.enable = flags & 1;
    c.probe = (flags >> 4) & 3;
    return NVFP4_OK;
}

}  // extern "C"

// Dense NVFP4 GEMM for more than two tokens (prefill, batched decode) on the 5th-generation
// tensor cores:  out[M, N] = dequant(W)[M, K] . act[K, N]   (N = tokens, act token-minor).
//
// Replaces the reference's wmma kernel behind the same entry point (kernels/nvfp4_cuda_v5.cu:188-399
// kernel, :406-422 launcher, caller pipeline/_qwen38_infer.py:174-181).  Arithmetic follows the
// reference (W4A16): a weight is decoded to fp16 and multiplied by its block scale IN fp16
// (kernels/nvfp4_cuda_v5.cu:163-175), products are fp16 x fp16, accumulation is fp32.
//
// Structure of one CTA (320 threads), tile = 128 weight rows x BN tokens, K in steps of 64:
//   warp 0        : TMA producer.  One elected thread issues cp.async.bulk.tensor.2d loads of the
//                   activation tile ([64 k] x [64 tokens] boxes, 128-byte swizzle) into a 4-stage
//                   shared-memory ring, completion on an mbarrier (transaction bytes).
//   warp 1        : MMA issuer.  One elected thread issues tcgen05.mma.kind::f16 (M = 128, N = BN,
//                   K = 16, four per stage) with shared-memory descriptors; the fp32 accumulator
//                   lives in tensor memory (BN columns).  tcgen05.commit releases each stage.
//   warps 2..9    : weight producers, two threads per weight row: 16 packed bytes + 2 scale bytes
//                   each per K step from global memory, nibbles -> fp16 (cvt.rn.f16x2.e2m1x2) x
//                   scale, written as a K-major, 128-byte-swizzled A tile; then the epilogue:
//                   tcgen05.ld of the accumulator (each warp its own 32-lane quarter and half of
//                   the token columns), fp16 store.
// A operand: K-major SWIZZLE_128B (row = 128 bytes = 64 fp16).  B operand: MN-major SWIZZLE_128B
// (one k row = 64 tokens = 128 bytes), exactly what the token-minor activation gives a TMA box.
//
// Every wait on an mbarrier is bounded: when the limit is reached the waiter records it in a
// device status word, stops waiting, and the CTA still runs to its end and frees its tensor
// memory, so a logic error can produce wrong numbers but never a hung GPU.
//
// Shapes the tensor-core kernel does not take (K % 64 != 0, N % 8 != 0, unaligned pointers) run
// on a plain CUDA-core kernel with the same arithmetic.
#include <cuda.h>

#include <cstdio>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace nvfp4 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_PRODUCER_WARPS = 8;   // weight-dequant warps (two threads per weight row)
constexpr int GEMM_THREADS = 64 + 32 * GEMM_PRODUCER_WARPS;
// K steps the weight loads run ahead of their use (8 measured 6 % slower at 8192 tokens; 16 for
// tiles of <= 64 tokens 11 % slower: those are bound by the one-thread roles' instruction latency,
// not by bytes in flight)
constexpr int GEMM_WPF = 4;
constexpr uint32_t GEMM_SPIN_LIMIT = 1u << 24;

__device__ int g_gemm_status = 0;  // 0 ok; otherwise 1 + id of the wait that ran out
static int g_gemm_rows256 = 1;     // 256-row CTA tiles for more than 128 tokens (0: 128-row tiles only)

// Bounded wait.  Returns false (after recording `id`) if the barrier never completed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int id) {
    for (uint32_t i = 0; i < GEMM_SPIN_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(&g_gemm_status, 1 + id);
    return false;
}
enum { GEMM_OUT_FM = 0, GEMM_OUT_TM = 1, GEMM_OUT_TM_ADD = 2 };   // output layouts, see the kernel

// Epilogue store of one 32-token block of a thread's row (v = 32 fp32 accumulator values), in the
// layout out_mode asks for.  m = this thread's row, mbase = first row of its 128-row tile,
// nb = first token of the block.  `piece` counts the token-major staging pieces of this column
// half (chalf); all four warps of a column half call this together.
__device__ __forceinline__ void gemm_store_block(const uint32_t (&v)[32], __half* out, int out_mode,
                                                 uint8_t* smem, int chalf, int& piece, int q, int lane,
                                                 int m, int mbase, int nb, int M, int N, int ld_out,
                                                 int n_out) {
    if (out_mode != GEMM_OUT_FM) {
        // Token-major: a thread holds one row's 32 tokens, memory wants one token's rows
        // together.  The four warps of this column half (128 rows) turn the 32 x 128 piece
        // over in shared memory - the operand ring is free once the accumulation has
        // retired - and then store 16 bytes (8 rows of one token) per thread.  Two staging
        // pieces alternate, so the one barrier per piece also orders a piece's writes
        // after the reads of the piece before last.  (Storing 2 bytes per lane straight
        // from the registers cost 4 us per 512-token GEMM, 23 us with the residual add.)
        __half* stg = reinterpret_cast<__half*>(smem + (chalf * 2 + (piece & 1)) * 8192);
        const int rr = q * 32 + lane;
#pragma unroll
        for (int j = 0; j < 32; j++) stg[j * 128 + rr] = __float2half(__uint_as_float(v[j]));
        asm volatile("bar.sync %0, 128;\n" ::"r"(1 + chalf) : "memory");
        const bool vec = ((ld_out & 7) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int pid = i * 128 + rr, tok = pid >> 4, part = pid & 15;
            const int tg = nb + tok, mg = mbase + part * 8;
            if (tg >= n_out || mg >= M) continue;
            const uint4 val = *reinterpret_cast<const uint4*>(stg + tok * 128 + part * 8);
            __half* p = out + (size_t)tg * (size_t)ld_out + mg;
            const __half2* h2 = reinterpret_cast<const __half2*>(&val);
            if (vec && mg + 8 <= M) {
                uint4 o = val;
                if (out_mode == GEMM_OUT_TM_ADD) {
                    const uint4 old = *reinterpret_cast<const uint4*>(p);
                    const __half2* r2 = reinterpret_cast<const __half2*>(&old);
                    __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 a = __half22float2(h2[e]), b = __half22float2(r2[e]);
                        o2[e] = __floats2half2_rn(a.x + b.x, a.y + b.y);
                    }
                }
                *reinterpret_cast<uint4*>(p) = o;
            } else {
                const __half* h1 = reinterpret_cast<const __half*>(&val);
                for (int e = 0; e < 8 && mg + e < M; e++) {
                    __half r = h1[e];
                    if (out_mode == GEMM_OUT_TM_ADD) r = __float2half(__half2float(r) + __half2float(p[e]));
                    p[e] = r;
                }
            }
        }
        piece++;
    } else if (m < M && nb < N) {
        __half* orow = out + (size_t)m * (size_t)N + nb;
        if (nb + 32 <= N) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint4 o;
                __half2 t;
                t = __floats2half2_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                o.x = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2half2_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                o.y = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2half2_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                o.z = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2half2_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                o.w = *reinterpret_cast<uint32_t*>(&t);
                *reinterpret_cast<uint4*>(orow + j) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (nb + j < N) orow[j] = __float2half(__uint_as_float(v[j]));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel.  BN = tokens per CTA tile (64, 128 or 256).
// Shared memory (dynamic, 1024-byte aligned): per stage A tile 128 x 128 B = 16 KB, then per stage
// B tile (BN/64) boxes of 64 k-rows x 128 B = 8 KB each.
// ---------------------------------------------------------------------------------------------
// MT = weight row tiles of 128 per CTA (1 or 2).  With MT = 2 a CTA computes 256 rows x BN tokens
// in two accumulators (2 x BN columns of tensor memory): the activation tile, which is most of the
// operand traffic from L2 (32 KB of the 36.5 KB a 128-row CTA pulls per K step at BN = 256), is
// fetched once for twice the rows.  The kernel was bound by that feed, not by the tensor pipe.
// IN_TM: the activations are token-major [tokens][K] (the layout the prefill keeps them in): one
// TMA box of BN tokens x 64 k per stage, a K-major B operand like the weights'.  Otherwise
// [K][tokens] as the reference's entry point takes them (an MN-major B operand).
// out_mode (run time): GEMM_OUT_FM out[m][token], row pitch N; GEMM_OUT_TM out[token][m], row pitch
// ld_out, tokens below n_out only (N may be padded to 8); GEMM_OUT_TM_ADD out[token][m] += result (the fp16-rounded result added in fp32, one more
// rounding: what a separate residual add of the fp16 output computes).
template <int BN, int MT, bool IN_TM>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_w4a16_tcgen05_kernel(const __grid_constant__ CUtensorMap act_map,
                          const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                          __half* out, int M, int N, int K, int ld_out, int out_mode, int n_out) {
    // (two stages and two CTAs per SM for the 256-token tile measured 8 % slower than this)
    constexpr int ST = (MT == 2 && BN == 256) ? 3 : GEMM_STAGES;
    constexpr int A_TILE = GEMM_BM * 128;           // 16 KB: one 128-row tile of a stage
    constexpr int A_BYTES = MT * A_TILE;
    constexpr int B_BOX = GEMM_BK * 128;            // 8 KB: 64 k rows of 64 tokens
    constexpr int B_BYTES = (BN / 64) * B_BOX;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the runtime aligns dynamic shared memory to 16 bytes only: round up to the swizzle atom
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + ST * A_BYTES;
    // one barrier per stage for both operands (256 dequantising threads arrive, the copy-issuing
    // thread arrives with the activation tile's byte count): the MMA-issuing thread runs one
    // instruction at a time, and a second wait per K step cost it as much as two MMAs
    __shared__ __align__(8) uint64_t bar_full[ST];
    __shared__ __align__(8) uint64_t bar_empty[ST];    // MMAs that read the stage retired
    __shared__ __align__(8) uint64_t bar_accum;                 // whole accumulation retired
    __shared__ uint32_t s_tmem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * GEMM_BM * MT, n0 = blockIdx.y * BN;
    const int ksteps = K / GEMM_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; s++) {
            mbar_init(smem_u32(&bar_full[s]), 32 * GEMM_PRODUCER_WARPS + 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_accum), 1);
        fence_barrier_init();
    }
    if (warp == 0) {  // one warp allocates the accumulator's tensor-memory columns
        tcgen05_alloc(smem_u32(&s_tmem), MT * BN);
        tcgen05_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = s_tmem;

    if (warp == 0) {
        // ---------------- TMA producer: activation tiles ----------------
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < ksteps && ok; it++) {
                const int s = it % ST;
                const uint32_t ph = (uint32_t)(it / ST) & 1u;
                ok = mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, 0);
                if (!ok) break;
                const uint32_t bar = smem_u32(&bar_full[s]);
                mbar_arrive_expect_tx(bar, B_BYTES);
                if constexpr (IN_TM) {
                    // x = element along K (64 fp16 = 128 bytes per step), y = token
                    tma_load_2d(smem_u32(smem_b + s * B_BYTES), &act_map, it * GEMM_BK, n0, bar);
                } else {
#pragma unroll
                    for (int b = 0; b < BN / 64; b++)
                        tma_load_2d(smem_u32(smem_b + s * B_BYTES + b * B_BOX), &act_map, n0 + b * 64,
                                    it * GEMM_BK, bar);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: D fp32, A fp16 K-major, B fp16 MN-major, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (IN_TM ? 0u : (1u << 16)) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)(GEMM_BM >> 4) << 24);
            // stage index, phase and operand addresses are kept by increment (no division, no
            // address arithmetic from scratch in this one-thread loop)
            int s = 0;
            uint32_t ph = 0;
            uint32_t a_base = smem_u32(smem_a), b_base = smem_u32(smem_b);
            uint32_t bar_f = smem_u32(&bar_full[0]), bar_e = smem_u32(&bar_empty[0]);
            for (int it = 0; it < ksteps; it++) {
                if (!mbar_wait(bar_f, ph, 1)) break;
                tcgen05_fence_after();
#pragma unroll
                for (int kk = 0; kk < GEMM_BK / 16; kk++) {
                    // A, K-major: 16 k = 32 bytes further along the 128-byte row; 8-row groups
                    // are 1024 bytes apart.  B, MN-major: 16 k = two groups of 8 k rows (1024
                    // bytes each); 64-token atoms are one box (8 KB) apart.
                    // (token-major activations: a K-major tile of BN token rows, like A)
                    const uint64_t bdesc = IN_TM ? make_desc_sw128(b_base + kk * 32, 16, 1024)
                                                 : make_desc_sw128(b_base + kk * 2048, B_BOX, 1024);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        const uint64_t adesc = make_desc_sw128(a_base + mt * A_TILE + kk * 32, 16, 1024);
                        tcgen05_mma_f16(tmem + (uint32_t)(mt * BN), adesc, bdesc, idesc,
                                        (it | kk) != 0 ? 1u : 0u);
                    }
                }
                tcgen05_commit(bar_e);                     // stage reusable when these MMAs retire
                a_base += A_BYTES; b_base += B_BYTES; bar_f += 8; bar_e += 8;
                if (++s == ST) {
                    s = 0; ph ^= 1u;
                    a_base = smem_u32(smem_a); b_base = smem_u32(smem_b);
                    bar_f = smem_u32(&bar_full[0]); bar_e = smem_u32(&bar_empty[0]);
                }
            }
            tcgen05_commit(smem_u32(&bar_accum));
        }
    } else {
        // ---------------- weight producers (two threads per weight row), then epilogue ----------------
        const int pt = threadIdx.x - 64;                 // 0..255
        const int r = pt >> 1, half = pt & 1;            // row of a 128-row tile, which 32 of its 64 weights
        const uint8_t* prow[MT];
        const uint8_t* srow[MT];
        bool row_ok[MT];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int rr = m0 + mt * GEMM_BM + r;
            row_ok[mt] = rr < M;
            const int row = min(rr, M - 1);
            prow[mt] = packed + (size_t)row * (size_t)(K >> 1) + half * 16;
            srow[mt] = scales + (size_t)row * (size_t)(K >> 4) + half * 2;
        }
        bool ok = true;
        // 16 packed bytes (32 weights = 2 scale blocks) per row and K step, requested GEMM_WPF steps
        // ahead of their use: the weight stream comes from HBM and its latency is longer than the
        // tensor core needs for one K step
        uint4 pw[GEMM_WPF][MT];
        uint32_t ps[GEMM_WPF][MT];
#pragma unroll
        for (int u = 0; u < GEMM_WPF; u++) {
            if (u < ksteps) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    pw[u][mt] = ld_stream_u4(prow[mt] + (size_t)u * 32);
                    ps[u][mt] = __ldg(reinterpret_cast<const unsigned short*>(srow[mt] + (size_t)u * 4));
                }
            }
        }
        for (int it0 = 0; it0 < ksteps; it0 += GEMM_WPF) {
#pragma unroll
        for (int u = 0; u < GEMM_WPF; u++) {
            const int it = it0 + u;
            if (it >= ksteps) break;
            const int s = it % ST;
            const uint32_t ph = (uint32_t)(it / ST) & 1u;
            uint4 p0[MT];
            uint32_t sc2[MT];
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                p0[mt] = pw[u][mt];
                sc2[mt] = ps[u][mt];
                if (it + GEMM_WPF < ksteps) {
                    pw[u][mt] = ld_stream_u4(prow[mt] + (size_t)(it + GEMM_WPF) * 32);
                    ps[u][mt] = __ldg(reinterpret_cast<const unsigned short*>(srow[mt] + (size_t)(it + GEMM_WPF) * 4));
                }
            }
            if (ok) ok = mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, 3);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const uint32_t w[4] = {p0[mt].x, p0[mt].y, p0[mt].z, p0[mt].w};
                uint8_t* arow = smem_a + s * A_BYTES + mt * A_TILE + r * 128;
#pragma unroll
                for (int j = 0; j < 4; j++) {               // 16-byte chunk c = weights 8c .. 8c+7
                    const int c = half * 4 + j;
                    uint32_t h0, h1, h2, h3;
                    e2m1x8_to_half2x4(w[j], h0, h1, h2, h3);
                    // block scale 2^(sb-127) as fp16, applied in fp16 as the reference does
                    const __half sc = __float2half(e8m0_to_f32((sc2[mt] >> (8 * (j >> 1))) & 0xFFu));
                    const __half2 s2 = __half2half2(sc);
                    uint4 v;
                    __half2 t;
                    t = __hmul2(*reinterpret_cast<__half2*>(&h0), s2); v.x = *reinterpret_cast<uint32_t*>(&t);
                    t = __hmul2(*reinterpret_cast<__half2*>(&h1), s2); v.y = *reinterpret_cast<uint32_t*>(&t);
                    t = __hmul2(*reinterpret_cast<__half2*>(&h2), s2); v.z = *reinterpret_cast<uint32_t*>(&t);
                    t = __hmul2(*reinterpret_cast<__half2*>(&h3), s2); v.w = *reinterpret_cast<uint32_t*>(&t);
                    if (!row_ok[mt]) v = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) << 4)) = v;   // 128-byte swizzle
                }
            }
            fence_proxy_async_smem();     // make the generic-proxy writes visible to the tensor core
            mbar_arrive(smem_u32(&bar_full[s]));
        }
        }

        // ---------------- epilogue: TMEM -> registers -> fp16 out[m][n] ----------------
        mbar_wait(smem_u32(&bar_accum), 0, 4);
        tcgen05_fence_after();
        const int q = warp & 3;                          // this warp's 32-lane quarter of TMEM
        const int chalf = (warp - 2) >> 2;               // which half of the token columns
        constexpr int CB = BN / 32;                      // 32-column blocks in the tile
        int piece = 0;
#pragma unroll 1
        for (int mt = 0; mt < MT; mt++) {
        const int m = m0 + mt * GEMM_BM + q * 32 + lane;
#pragma unroll
        for (int cbi = 0; cbi < (CB + 1) / 2; cbi++) {
            const int cb = chalf * ((CB + 1) / 2) + cbi;
            if (cb >= CB) break;
            uint32_t v[32];
            tcgen05_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * BN + cb * 32), v);
            tcgen05_wait_ld();
            const int nb = n0 + cb * 32;
            gemm_store_block(v, out, out_mode, smem, chalf, piece, q, lane, m, m0 + mt * GEMM_BM, nb, M, N,
                             ld_out, n_out);
        }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tcgen05_dealloc(tmem, MT * BN);
}

// ---------------------------------------------------------------------------------------------
// CTA-pair kernel (cluster of two, tcgen05 cta_group::2): 256 weight rows x 256 tokens per pair.
// Each CTA dequantises its own 128 rows (A tile, 16 KB per K step) and loads HALF of the token
// tile (128 tokens, 16 KB); one thread of the pair's first CTA issues M = 256 MMAs that run on both
// SMs' tensor cores, each reading its own A rows and both halves of B.  Per SM and K step that is
// 20.5 KB from L2 instead of 36.5 KB (the measured ingest limit of an SM is about 41 bytes per
// clock, which held a 128-row x 256-token CTA at 880 cycles per step against 512 of MMA time) and
// 64 KB instead of 96 KB through shared memory; the ring is 3 stages of 64 KB (two K steps each).
// Barriers live at the same offsets in both CTAs.  full[s] is used in the first CTA only: one
// arrival per dequantising warp of either CTA (after the warp's lanes fenced their writes) and one
// arrive-with-byte-count per copy-issuing thread, the peer's through shared::cluster addresses;
// empty[s] and accum are committed to in each CTA separately.
// ---------------------------------------------------------------------------------------------
// A stage holds PAIR_KS K steps (128 elements of K): the thread that issues the MMAs pays one wait
// and the commits per stage, and with one K step per stage those cost it more than the MMAs.
constexpr int PAIR_BN = 256, PAIR_HALF = 128, PAIR_ST = 3, PAIR_KS = 2;
// Bounded wait on a barrier that the peer CTA (or a commit issued there) arrives on.
__device__ __forceinline__ bool pair_wait(uint32_t bar, uint32_t parity, int id) {
    for (uint32_t i = 0; i < GEMM_SPIN_LIMIT; i++)
        if (mbar_test_wait_cluster(bar, parity)) return true;
    atomicExch(&g_gemm_status, 1 + id);
    return false;
}
template <bool IN_TM>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_w4a16_pair_kernel(const __grid_constant__ CUtensorMap act_map,
                       const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                       __half* out, int M, int N, int K, int ld_out, int out_mode, int n_out) {
    constexpr int ST = PAIR_ST;
    constexpr int KS = PAIR_KS;
    constexpr int A_SUB = GEMM_BM * 128;            // 16 KB: 128 rows x one K step
    constexpr int A_BYTES = KS * A_SUB;             // a stage of A
    constexpr int B_BOX = GEMM_BK * 128;            // 8 KB: 64 k rows of 64 tokens (token-minor input)
    constexpr int B_SUB = PAIR_HALF * 128;          // 16 KB: this CTA's half of the token tile, one K step
    constexpr int B_BYTES = KS * B_SUB;
    constexpr int BN = PAIR_BN;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + ST * A_BYTES;
    __shared__ __align__(8) uint64_t bar_full[ST];
    __shared__ __align__(8) uint64_t bar_empty[ST];
    __shared__ __align__(8) uint64_t bar_accum;
    __shared__ uint32_t s_tmem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();        // 0 = the CTA that issues the MMAs
    const int m0 = blockIdx.x * GEMM_BM;             // blockIdx.x = 2 * pair + rank
    const int n0 = blockIdx.y * BN;
    const int nh = n0 + (int)rank * PAIR_HALF;       // first token of this CTA's half of B
    const int ksteps = K / GEMM_BK;              // a multiple of KS (the launcher checks)
    const int nstages = ksteps / KS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; s++) {
            mbar_init(smem_u32(&bar_full[s]), 2 * GEMM_PRODUCER_WARPS + 2);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_accum), 1);
        fence_barrier_init();
    }
    if (warp == 0) {   // the same warp of both CTAs allocates the pair's accumulator columns
        tcgen05_alloc_pair(smem_u32(&s_tmem), BN);
        tcgen05_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();      // the peer's barriers are initialised before anything arrives on them
    tcgen05_fence_after();
    const uint32_t tmem = s_tmem;

    if (warp == 0) {
        // ---------------- TMA producer: this CTA's half of the activation tile ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (int st = 0; st < nstages; st++) {
                if (!pair_wait(smem_u32(&bar_empty[s]), ph ^ 1u, 0)) break;
                const uint32_t bar = cluster_map_shared(smem_u32(&bar_full[s]), 0);
                mbar_arrive_expect_tx_cluster(bar, B_BYTES);
#pragma unroll
                for (int h = 0; h < KS; h++) {
                    const int it = st * KS + h;
                    const uint32_t dst = smem_u32(smem_b + s * B_BYTES + h * B_SUB);
                    if constexpr (IN_TM) {
                        tma_load_2d_pair(dst, &act_map, it * GEMM_BK, nh, bar);
                    } else {
#pragma unroll
                        for (int b = 0; b < PAIR_HALF / 64; b++)
                            tma_load_2d_pair(dst + b * B_BOX, &act_map, nh + b * 64, it * GEMM_BK, bar);
                    }
                }
                if (++s == ST) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: first CTA of the pair only ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (IN_TM ? 0u : (1u << 16)) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)((2 * GEMM_BM) >> 4) << 24);
            int s = 0;
            uint32_t ph = 0;
            uint32_t a_base = smem_u32(smem_a), b_base = smem_u32(smem_b);
            for (int st = 0; st < nstages; st++) {
                if (!pair_wait(smem_u32(&bar_full[s]), ph, 5)) break;
                tcgen05_fence_after();
#pragma unroll
                for (int h = 0; h < KS; h++) {
#pragma unroll
                    for (int kk = 0; kk < GEMM_BK / 16; kk++) {
                        const uint64_t adesc = make_desc_sw128(a_base + h * A_SUB + kk * 32, 16, 1024);
                        const uint64_t bdesc = IN_TM ? make_desc_sw128(b_base + h * B_SUB + kk * 32, 16, 1024)
                                                     : make_desc_sw128(b_base + h * B_SUB + kk * 2048, B_BOX, 1024);
                        tcgen05_mma_f16_pair(tmem, adesc, bdesc, idesc, (st | h | kk) != 0 ? 1u : 0u);
                    }
                }
                // the stage is free in both CTAs once these MMAs have retired
                const uint32_t be = smem_u32(&bar_empty[s]);
                tcgen05_commit_pair(cluster_map_shared(be, 0));
                tcgen05_commit_pair(cluster_map_shared(be, 1));
                a_base += A_BYTES; b_base += B_BYTES;
                if (++s == ST) { s = 0; ph ^= 1u; a_base = smem_u32(smem_a); b_base = smem_u32(smem_b); }
            }
            const uint32_t ba = smem_u32(&bar_accum);
            tcgen05_commit_pair(cluster_map_shared(ba, 0));
            tcgen05_commit_pair(cluster_map_shared(ba, 1));
        }
    } else {
        // ---------------- weight producers (two threads per weight row), then epilogue ----------------
        const int pt = threadIdx.x - 64;
        const int r = pt >> 1, half = pt & 1;
        const int rr0 = m0 + r;
        const bool row_ok = rr0 < M;
        const int row = min(rr0, M - 1);
        const uint8_t* prow = packed + (size_t)row * (size_t)(K >> 1) + half * 16;
        const uint8_t* srow = scales + (size_t)row * (size_t)(K >> 4) + half * 2;
        bool ok = true;
        uint4 pw[GEMM_WPF];
        uint32_t ps[GEMM_WPF];
#pragma unroll
        for (int u = 0; u < GEMM_WPF; u++) {
            if (u < ksteps) {
                pw[u] = ld_stream_u4(prow + (size_t)u * 32);
                ps[u] = __ldg(reinterpret_cast<const unsigned short*>(srow + (size_t)u * 4));
            }
        }
        int s = 0;
        uint32_t ph = 0;
        for (int it0 = 0; it0 < ksteps; it0 += GEMM_WPF) {
#pragma unroll
        for (int u = 0; u < GEMM_WPF; u++) {
            const int it = it0 + u;
            if (it >= ksteps) break;
            const uint4 p0 = pw[u];
            const uint32_t sc2 = ps[u];
            if (it + GEMM_WPF < ksteps) {
                pw[u] = ld_stream_u4(prow + (size_t)(it + GEMM_WPF) * 32);
                ps[u] = __ldg(reinterpret_cast<const unsigned short*>(srow + (size_t)(it + GEMM_WPF) * 4));
            }
            if ((u & (KS - 1)) == 0 && ok) ok = pair_wait(smem_u32(&bar_empty[s]), ph ^ 1u, 3);
            const uint32_t w[4] = {p0.x, p0.y, p0.z, p0.w};
            uint8_t* arow = smem_a + s * A_BYTES + (u & (KS - 1)) * A_SUB + r * 128;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int c = half * 4 + j;
                uint32_t h0, h1, h2, h3;
                e2m1x8_to_half2x4(w[j], h0, h1, h2, h3);
                const __half sc = __float2half(e8m0_to_f32((sc2 >> (8 * (j >> 1))) & 0xFFu));
                const __half2 s2 = __half2half2(sc);
                uint4 v;
                __half2 t;
                t = __hmul2(*reinterpret_cast<__half2*>(&h0), s2); v.x = *reinterpret_cast<uint32_t*>(&t);
                t = __hmul2(*reinterpret_cast<__half2*>(&h1), s2); v.y = *reinterpret_cast<uint32_t*>(&t);
                t = __hmul2(*reinterpret_cast<__half2*>(&h2), s2); v.z = *reinterpret_cast<uint32_t*>(&t);
                t = __hmul2(*reinterpret_cast<__half2*>(&h3), s2); v.w = *reinterpret_cast<uint32_t*>(&t);
                if (!row_ok) v = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) << 4)) = v;
            }
            if ((u & (KS - 1)) == KS - 1) {
                fence_proxy_async_smem();     // each lane's writes, for the tensor cores' reads
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(cluster_map_shared(smem_u32(&bar_full[s]), 0));
                if (++s == ST) { s = 0; ph ^= 1u; }
            }
        }
        }

        // ---------------- epilogue: this CTA's 128 rows x 256 tokens ----------------
        pair_wait(smem_u32(&bar_accum), 0, 4);
        tcgen05_fence_after();
        const int q = warp & 3;
        const int chalf = (warp - 2) >> 2;
        constexpr int CB = BN / 32;
        int piece = 0;
        const int m = m0 + q * 32 + lane;
#pragma unroll 1
        for (int cbi = 0; cbi < CB / 2; cbi++) {
            const int cb = chalf * (CB / 2) + cbi;
            uint32_t v[32];
            tcgen05_ld_32x32b_x32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb * 32), v);
            tcgen05_wait_ld();
            const int nb = n0 + cb * 32;
            gemm_store_block(v, out, out_mode, smem, chalf, piece, q, lane, m, m0, nb, M, N, ld_out, n_out);
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();      // neither CTA leaves (or frees tensor memory) while the other may still use it
    if (warp == 0) tcgen05_dealloc_pair(tmem, BN);
}

// ---------------------------------------------------------------------------------------------
// CUDA-core fallback: any K % 16 == 0, any N, any alignment.  One thread per output, same
// arithmetic (weight x scale in fp16, fp32 accumulation).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gemm_w4a16_fallback_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                           const __half* __restrict__ act, __half* __restrict__ out, int M, int N,
                           int K) {
    const int n = blockIdx.x * 64 + (threadIdx.x & 63);
    const int m = blockIdx.y * 4 + (threadIdx.x >> 6);
    if (m >= M || n >= N) return;
    const uint8_t* prow = packed + (size_t)m * (size_t)(K >> 1);
    const uint8_t* srow = scales + (size_t)m * (size_t)(K >> 4);
    float acc = 0.0f;
    for (int b = 0; b < (K >> 4); b++) {
        const __half sc = __float2half(e8m0_to_f32(srow[b]));
        for (int i = 0; i < 8; i++) {
            const uint32_t h = e2m1x2_to_half2(prow[b * 8 + i]);
            const __half2 w = __hmul2(*reinterpret_cast<const __half2*>(&h), __half2half2(sc));
            const int k = b * 16 + 2 * i;
            acc = fmaf(__low2float(w), __half2float(act[(size_t)k * N + n]), acc);
            acc = fmaf(__high2float(w), __half2float(act[(size_t)(k + 1) * N + n]), acc);
        }
    }
    out[(size_t)m * N + n] = __float2half(acc);
}

template <int BN, int MT, bool IN_TM>
static cudaError_t launch_tc(const CUtensorMap& map, const uint8_t* packed, const uint8_t* scales,
                             __half* out, int M, int N, int K, int ld_out, int out_mode, int n_out,
                             cudaStream_t st) {
    constexpr int ST = (MT == 2 && BN == 256) ? 3 : GEMM_STAGES;
    constexpr int SMEM = ST * (MT * GEMM_BM * 128 + (BN / 64) * GEMM_BK * 128) + 1024;
    static bool attr[NVFP4_MAX_DEVICES] = {false};   // the attribute is per device
    const int dev = current_device_index();
    if (!attr[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_w4a16_tcgen05_kernel<BN, MT, IN_TM>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        attr[dev] = true;
    }
    dim3 grid((unsigned)((M + GEMM_BM * MT - 1) / (GEMM_BM * MT)), (unsigned)((N + BN - 1) / BN));
    gemm_w4a16_tcgen05_kernel<BN, MT, IN_TM><<<grid, GEMM_THREADS, SMEM, st>>>(map, packed, scales, out, M, N,
                                                                             K, ld_out, out_mode, n_out);
    return cudaGetLastError();
}

// The CTA-pair kernel: grid.x = 2 CTAs per 256 rows, launched as clusters of two along x.
static int g_gemm_pair = 1;        // 1: the CTA-pair kernel where 256-row tiles are not used; 2: wherever it can run
template <bool IN_TM>
static cudaError_t launch_pair(const CUtensorMap& map, const uint8_t* packed, const uint8_t* scales,
                               __half* out, int M, int N, int K, int ld_out, int out_mode, int n_out,
                               cudaStream_t st) {
    constexpr int SMEM = PAIR_ST * PAIR_KS * (GEMM_BM * 128 + PAIR_HALF * 128) + 1024;
    static bool attr[NVFP4_MAX_DEVICES] = {false};
    const int dev = current_device_index();
    if (!attr[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_w4a16_pair_kernel<IN_TM>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        attr[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * ((M + 255) / 256)), (unsigned)((N + PAIR_BN - 1) / PAIR_BN), 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_w4a16_pair_kernel<IN_TM>, map, packed, scales, out, M, N, K, ld_out,
                              out_mode, n_out);
}
// Tile choice, shared by both entry points.  Wider token tiles amortise the weight dequantisation
// over more tensor-core work; 256-row tiles when they still give every SM a CTA (17408 x 512
// tokens: 136 CTAs, 1282 TFLOP/s against 967 with 128-row tiles; 6144 x 512: 48 CTAs, slower).
static int gemm_tile_bn(int N) { return N > 128 ? 256 : N > 64 ? 128 : 64; }
static bool gemm_tile_rows256(int M, int N) {
    return N > 128 && g_gemm_rows256 && (long long)((M + 255) / 256) * ((N + 255) / 256) >= 120;
}
// The CTA-pair kernel takes more than 128 tokens and K % 128 == 0.  Measured at 512 tokens against
// the single-CTA kernel's best tile: 5120 x 5120 36.4 us (40.4), 6144 x 5120 38.4 (42.0), 10240 x
// 5120 69.4 (77.2), 5120 x 17408 105.7 (121.0) - but 17408 x 5120 75.6 (69.3 with 256-row tiles) and
// 34816 x 5120 149 (140): it replaces the 128-row tiles, not the 256-row ones.
static bool gemm_use_pair(int M, int N, int K) {
    if (!g_gemm_pair || N <= 128 || K % (GEMM_BK * PAIR_KS) != 0) return false;
    return g_gemm_pair == 2 || !gemm_tile_rows256(M, N);
}
template <bool IN_TM>
static cudaError_t launch_tc_any(const CUtensorMap& map, const uint8_t* packed, const uint8_t* scales,
                                 __half* out, int M, int N, int K, int ld_out, int out_mode, int n_out,
                                 cudaStream_t st) {
    if (gemm_use_pair(M, N, K)) return launch_pair<IN_TM>(map, packed, scales, out, M, N, K, ld_out, out_mode, n_out, st);
    return gemm_tile_rows256(M, N) ? launch_tc<256, 2, IN_TM>(map, packed, scales, out, M, N, K, ld_out, out_mode, n_out, st)
         : (N > 128)               ? launch_tc<256, 1, IN_TM>(map, packed, scales, out, M, N, K, ld_out, out_mode, n_out, st)
         : (N > 64)                ? launch_tc<128, 1, IN_TM>(map, packed, scales, out, M, N, K, ld_out, out_mode, n_out, st)
                                   : launch_tc<64, 1, IN_TM>(map, packed, scales, out, M, N, K, ld_out, out_mode, n_out, st);
}

}  // namespace nvfp4

extern "C" {

// out[M, N] (fp16) = dequant(W)[M, K] . act[K, N] (fp16, token-minor).  Returns 0 or the
// cudaError_t of the launch, as the reference does; -2 for a shape no kernel takes (K % 16 != 0,
// non-positive sizes, NULL pointers).
int launch_nvfp4_gemmtc_v5(const uint8_t* d_weight_packed, const uint8_t* d_weight_scales,
                           const void* d_activation_v, void* d_output_v, int M, int N, int K,
                           void* stream) {
    using namespace nvfp4;
    // the header is plain C: fp16 pointers travel as void* (the reference declares __half*)
    const __half* d_activation = static_cast<const __half*>(d_activation_v);
    __half* d_output = static_cast<__half*>(d_output_v);
    if (M <= 0 || N <= 0 || K <= 0 || K % 16 != 0) return NVFP4_ERR_SHAPE;
    if (!d_weight_packed || !d_weight_scales || !d_activation || !d_output) return NVFP4_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const bool tc_ok = (K % 64 == 0) && (N % 8 == 0) &&
                       (((uintptr_t)d_weight_packed & 15) == 0) &&
                       (((uintptr_t)d_weight_scales & 3) == 0) &&
                       (((uintptr_t)d_activation & 15) == 0) && (((uintptr_t)d_output & 15) == 0);
    EncodeTiledFn enc = tc_ok ? encode_tiled_fn() : nullptr;
    if (enc) {
        CUtensorMap map;
        const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};        // inner = tokens
        const cuuint64_t strides[1] = {(cuuint64_t)N * sizeof(__half)};   // bytes between k rows
        const cuuint32_t box[2] = {64, (cuuint32_t)GEMM_BK};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)d_activation, dims,
                               strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS) {
            const cudaError_t e = launch_tc_any<false>(map, d_weight_packed, d_weight_scales, d_output, M,
                                                       N, K, N, GEMM_OUT_FM, N, st);
            return (e == cudaSuccess) ? 0 : (int)e;
        }
    }
    dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 3) / 4));
    gemm_w4a16_fallback_kernel<<<grid, 256, 0, st>>>(d_weight_packed, d_weight_scales, d_activation,
                                                     d_output, M, N, K);
    const cudaError_t e = cudaGetLastError();
    return (e == cudaSuccess) ? 0 : (int)e;
}

// The same product with the layouts a token-major caller (the chunked prefill) has and wants:
//   flags bit 0: activations token-major act[n_tokens][ld_act] (else act[K][ld_act], tokens minor)
//   flags bit 1: output token-major out[n_tokens][ld_out] (else out[M][ld_out])
//   flags bit 2 (with bit 1): out[t][m] += result - the residual add of the reference's decoder
//                layer, computed as a separate fp16 add of the rounded GEMM output would
// Tensor-core kernel only: K % 64 == 0, ld_act % 8 == 0, 16-byte aligned pointers, feature-major
// sides need ld == n_tokens rounded up to 8.  0; -2 for anything else (callers then transpose and use
// launch_nvfp4_gemmtc_v5); -3 without a tensor-map encoder; or the launch's cudaError_t.
int launch_nvfp4_gemm_w4a16_ex(const uint8_t* d_weight_packed, const uint8_t* d_weight_scales,
                               const void* act, long long ld_act, void* out, long long ld_out, int M,
                               int n_tokens, int K, int flags, void* stream) {
    using namespace nvfp4;
    if (M <= 0 || n_tokens <= 0 || K <= 0 || K % 64 != 0 || (flags & ~7) != 0) return NVFP4_ERR_SHAPE;
    if (!d_weight_packed || !d_weight_scales || !act || !out) return NVFP4_ERR_SHAPE;
    const bool in_tm = flags & 1, out_tm = flags & 2, add = flags & 4;
    if (add && !out_tm) return NVFP4_ERR_SHAPE;
    const int N8 = (n_tokens + 7) / 8 * 8;
    if (ld_act % 8 != 0 || ld_act < (in_tm ? K : n_tokens) || ld_act > 0x7fffffffLL) return NVFP4_ERR_SHAPE;
    if (!in_tm && ld_act != N8) return NVFP4_ERR_SHAPE;
    if (out_tm ? (ld_out < M) : (ld_out != N8)) return NVFP4_ERR_SHAPE;
    if (ld_out > 0x7fffffffLL) return NVFP4_ERR_SHAPE;
    if ((((uintptr_t)d_weight_packed | (uintptr_t)act) & 15) != 0 || ((uintptr_t)d_weight_scales & 3) != 0 ||
        ((uintptr_t)out & (out_tm ? 1 : 15)) != 0)
        return NVFP4_ERR_SHAPE;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return -3;
    // token count the kernel's bounds use: feature-major sides are padded to 8
    const int N = (in_tm && out_tm) ? n_tokens : N8;
    CUtensorMap map;
    const cuuint32_t estr[2] = {1, 1};
    CUresult r;
    if (in_tm) {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)n_tokens};       // inner = K
        const cuuint64_t strides[1] = {(cuuint64_t)ld_act * sizeof(__half)};
        const cuuint32_t box[2] = {(cuuint32_t)GEMM_BK,
                                   (cuuint32_t)(gemm_use_pair(M, N, K) ? PAIR_HALF : gemm_tile_bn(N))};
        r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(act), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const cuuint64_t dims[2] = {(cuuint64_t)N8, (cuuint64_t)K};
        const cuuint64_t strides[1] = {(cuuint64_t)N8 * sizeof(__half)};
        const cuuint32_t box[2] = {64, (cuuint32_t)GEMM_BK};
        r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(act), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return -3;
    const int mode = !out_tm ? GEMM_OUT_FM : add ? GEMM_OUT_TM_ADD : GEMM_OUT_TM;
    __half* o = static_cast<__half*>(out);
    cudaStream_t st = (cudaStream_t)stream;
    const cudaError_t e = in_tm ? launch_tc_any<true>(map, d_weight_packed, d_weight_scales, o, M, N, K,
                                                      (int)ld_out, mode, n_tokens, st)
                                : launch_tc_any<false>(map, d_weight_packed, d_weight_scales, o, M, N, K,
                                                       (int)ld_out, mode, n_tokens, st);
    return (e == cudaSuccess) ? 0 : (int)e;
}

// W4A4 product with the reference format on both sides: out[M, N] = dequant(W) .
// dequant(quant(act))^T, activations token-major [n_tokens][K] fp16, quantised per 16-element
// block along K by the codec's rule.  work: scratch of K * N fp16 elements, N = n_tokens rounded
// up to a multiple of 8 = the row length of `out`.
// K % 256 == 0 and aligned pointers: the activations are encoded to NVFP4 bytes in `work`
// (launch_nvfp4_encode) and the product runs on the block-scaled FP4 tensor-core path
// (launch_nvfp4_gemm_fp4); nothing is expanded to fp16.  Other shapes: launch_nvfp4_quant_dequant_T
// into work, then the W4A16 tensor-core GEMM (fp16 holds every FP4 value times its scale exactly;
// fp32 accumulation).  0, -2 for bad arguments, or a launch error code.
int launch_nvfp4_gemm_w4a4(const uint8_t* d_weight_packed, const uint8_t* d_weight_scales,
                           const void* d_activation, void* d_output, void* work, int M,
                           int n_tokens, int K, void* stream) {
    if (!work || n_tokens <= 0 || M <= 0 || K <= 0 || K % 16 != 0) return NVFP4_ERR_SHAPE;
    const int N = (n_tokens + 7) / 8 * 8;
    if (K % 256 == 0 && (((uintptr_t)work | (uintptr_t)d_activation) & 15) == 0) {
        uint8_t* a_packed = static_cast<uint8_t*>(work);
        const size_t pbytes = ((size_t)n_tokens * (size_t)(K / 2) + 255) & ~(size_t)255;
        uint8_t* a_scales = a_packed + pbytes;
        int rc = launch_nvfp4_encode(d_activation, a_packed, a_scales, n_tokens, K, stream);
        if (rc == 0) {
            rc = launch_nvfp4_gemm_fp4(d_weight_packed, d_weight_scales, a_packed, a_scales, d_output,
                                       M, n_tokens, K, N, stream);
            if (rc != NVFP4_ERR_SHAPE && rc != -3) return rc;
        } else if (rc != NVFP4_ERR_SHAPE) {
            return rc;
        }
    }
    const int rc = launch_nvfp4_quant_dequant_T(d_activation, K, work, N, n_tokens, K, stream);
    if (rc != 0) return rc;
    return launch_nvfp4_gemmtc_v5(d_weight_packed, d_weight_scales, work, d_output, M, N, K,
                                  stream);
}

// 0 if no bounded wait inside the tensor-core GEMMs (W4A16 and FP4) has run out since the library was loaded (or
// since the last call with reset != 0); otherwise 1 + the id of the wait.  Synchronises the device.
int nvfp4_gemm_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, nvfp4::g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    if (reset) {
        const int z = 0;
        cudaMemcpyToSymbol(nvfp4::g_gemm_status, &z, sizeof(int));
    }
    const int f = nvfp4_gemm_fp4_status(reset);   // the FP4 kernel's waits: ids 100 + its own
    if (v == 0 && f != 0) v = (f < 0) ? f : 100 + f;
    return v;
}

// Tuning hook.  Bit 0: 256-row CTA tiles (two accumulators) for more than 128 tokens.  Bit 1: the
// CTA-pair kernel (clusters of two, cta_group::2) for shapes of more than 128 tokens that do not get
// 256-row tiles.  Bit 2: the CTA-pair kernel for every shape it can run.  Default 3.
void nvfp4_b200_gemm_config(int flags) {
    nvfp4::g_gemm_rows256 = (flags & 1) ? 1 : 0;
    nvfp4::g_gemm_pair = (flags & 4) ? 2 : (flags & 2) ? 1 : 0;
}

// Shared memory of the tensor-core GEMM's widest tile, for callers that size their launches the
// way the reference's get_kernel_shared_mem_bytes does (kernels/nvfp4_cuda_v5.cu:460-464).
int get_kernel_shared_mem_bytes() {
    return 3 * (2 * nvfp4::GEMM_BM * 128 + 4 * nvfp4::GEMM_BK * 128) + 1024;
}

}  // extern "C"

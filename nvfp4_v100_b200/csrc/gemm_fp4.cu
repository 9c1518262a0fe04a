// W4A4 GEMM on the block-scaled FP4 tensor-core path:
//   out[M, ld_out] (fp16) = dequant(W)[M, K] . dequant(A)[n_tokens, K]^T
// Both operands stay in the container's format all the way into the tensor core: E2M1 nibbles, two
// per byte (low nibble = even element), one E8M0 scale byte per 16 elements along K
// (codec/nvfp4_codec.py:13-19 layout, :60-86 decode rule).  No fp16 copy of either operand is made;
// tcgen05.mma kind::mxf4nvf4 with 16-element scale blocks multiplies the nibbles, applies both block
// scales and accumulates in fp32 in tensor memory.  This is the FP4 path the reference names as its
// aim for tensor cores that have it (README.md "W4A4", kernels/nvfp4_cuda_v5.cu:1-20 keeps W4A16
// because its target GPU has none).
//
// One CTA (192 threads) computes a 128-row x BN-token tile, K in stages of 256 elements:
//   warp 0      TMA producer: per stage one box of weight bytes (128 rows x 128 B) and one box of
//               activation bytes (BN tokens x 128 B), both K-major with the 128-byte swizzle, and the
//               two boxes of their scale bytes (rows x 16 B), into an ST-stage shared-memory ring;
//               completion by transaction bytes on an mbarrier.
//   warp 1      MMA issuer: 4 tcgen05.mma (K = 64 each) per stage, one elected thread;
//               tcgen05.commit hands the stage back.
//   warps 2..5  scale-factor writers, then the epilogue.  The tensor core reads the scale bytes from
//               tensor memory: for an operand row r (weight row or token) of the tile, lane r % 32,
//               32-bit column r / 32 holds the row's 4 scale bytes of one 64-element K block, the
//               same in all four 32-lane quarters.  Each of the 4 warps owns one quarter: a lane
//               reads 16 scale bytes (one stage) of each of its rows from the ring and writes
//               them with tcgen05.st.  Per stage 16 columns for the weights and max(BN / 8, 16) for the tokens.
// Tensor memory: BN accumulator columns + ST x (16 + max(BN/8, 16)) scale columns.
//
// Every wait is bounded (status word, see nvfp4_gemm_fp4_status); a CTA always runs to its end and
// frees its tensor memory.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace nvfp4 {

constexpr int F4_BM = 128;
constexpr int F4_BK = 256;                 // elements of K per stage = 128 bytes per row
constexpr int F4_THREADS = 192;
constexpr int F4_PAIR_THREADS = 320;       // the CTA-pair kernel: two sets of scale-writing warps
constexpr uint32_t F4_SPIN_LIMIT = 1u << 24;

__device__ int g_fp4_status = 0;           // 0 ok; otherwise 1 + id of the wait that ran out

__device__ __forceinline__ bool f4_wait(uint32_t bar, uint32_t parity, int id) {
    for (uint32_t i = 0; i < F4_SPIN_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(&g_fp4_status, 1 + id);
    return false;
}

__device__ __forceinline__ void tcgen05_mma_fp4_block16(uint32_t taddr, uint64_t adesc, uint64_t bdesc,
                                                        uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                        uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::
            "r"(taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
// Non-suspending poll: for barriers that the peer CTA of a pair, or a commit issued there, arrives on.
__device__ __forceinline__ bool f4_wait_poll(uint32_t bar, uint32_t parity, int id) {
    for (uint32_t i = 0; i < F4_SPIN_LIMIT; i++)
        if (mbar_test_wait_cluster(bar, parity)) return true;
    atomicExch(&g_fp4_status, 1 + id);
    return false;
}
__device__ __forceinline__ void tcgen05_mma_fp4_block16_pair(uint32_t taddr, uint64_t adesc, uint64_t bdesc,
                                                             uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                             uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::
            "r"(taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ void tcgen05_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
// tcgen05.st, shape 32x32b: lane l of the warp writes NR consecutive 32-bit columns of its own lane
template <int NR>
__device__ __forceinline__ void tcgen05_st_32x32b(uint32_t taddr, const uint32_t* r) {
    static_assert(NR == 1 || NR == 2 || NR == 4 || NR == 8, "column count");
    if constexpr (NR == 1)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};\n" ::"r"(taddr), "r"(r[0]) : "memory");
    else if constexpr (NR == 2)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1,%2};\n" ::"r"(taddr), "r"(r[0]),
                     "r"(r[1]) : "memory");
    else if constexpr (NR == 4)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(taddr), "r"(r[0]),
                     "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
    else
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"r"(taddr),
                     "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                     : "memory");
}

__host__ __device__ constexpr int f4_tmem_cols(int need) { return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512; }

template <int BN, int ST>
__global__ void __launch_bounds__(F4_THREADS)
gemm_fp4_block_scaled_kernel(const __grid_constant__ CUtensorMap w_map,
                             const __grid_constant__ CUtensorMap a_map,
                             const __grid_constant__ CUtensorMap ws_map,
                             const __grid_constant__ CUtensorMap as_map,
                             __half* __restrict__ out, int M, int n_tokens, int K, int ld_out,
                             float* __restrict__ part, unsigned int* __restrict__ counters, int kper) {
    constexpr int A_BYTES = F4_BM * 128;             // weight tile of a stage
    constexpr int B_BYTES = BN * 128;                // token tile of a stage
    constexpr int NB = BN / 32;                      // token rows per lane
    // one MMA's scale bytes start on a 4-column boundary of tensor memory (an address between
    // boundaries raised "misaligned address"), so narrow token tiles leave columns unused
    constexpr int NBC = NB < 4 ? 4 : NB;             // token-scale columns reserved per MMA
    constexpr int SFA_COLS = 16, SFB_COLS = 4 * NBC, SF_COLS = SFA_COLS + SFB_COLS;
    constexpr int TCOLS = f4_tmem_cols(BN + ST * SF_COLS);
    static_assert(BN + ST * SF_COLS <= 512, "tensor memory");
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~(uintptr_t)1023);
    constexpr int SA_BYTES = F4_BM * 16;             // weight scale bytes of a stage
    constexpr int SB_BYTES = BN * 16;                // token scale bytes of a stage
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + ST * A_BYTES;
    uint8_t* smem_sa = smem_b + ST * B_BYTES;
    uint8_t* smem_sb = smem_sa + ST * SA_BYTES;
    __shared__ __align__(8) uint64_t bar_full[ST];    // TMA bytes landed
    __shared__ __align__(8) uint64_t bar_sf[ST];      // scale bytes written to tensor memory
    __shared__ __align__(8) uint64_t bar_empty[ST];   // the stage's MMAs retired
    __shared__ __align__(8) uint64_t bar_accum;       // a tile's accumulation retired
    __shared__ __align__(8) uint64_t bar_acc_free;    // the epilogue has read the accumulator
    __shared__ uint32_t s_tmem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // A CTA walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ... (row tile fastest): barriers,
    // tensor memory and the tensor maps are set up once, and the copies of the next tile's first
    // stages run under this tile's epilogue.  With a K split (gridDim.z > 1) the grid has one
    // CTA per tile and split.
    const int tiles_m = (M + F4_BM - 1) / F4_BM;
    const int ntiles = tiles_m * ((n_tokens + BN - 1) / BN);
    // K split (gridDim.z > 1; few CTA tiles, e.g. 32 tokens x 5120 rows): this CTA takes the stages
    // [k_first, k_first + ksteps) and the tile's CTAs meet in the epilogue
    const int k_first = (int)blockIdx.z * kper;
    const int ksteps = min(kper, K / F4_BK - k_first);
    __shared__ int s_last;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; s++) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_sf[s]), 128);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_accum), 1);
        mbar_init(smem_u32(&bar_acc_free), 128);
        fence_barrier_init();
    }
    if (warp == 0) {
        tcgen05_alloc(smem_u32(&s_tmem), TCOLS);
        tcgen05_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmem_sf = tmem + BN;               // scale columns follow the accumulator

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * F4_BM, n0 = (tile / tiles_m) * BN;
                for (int it = 0; it < ksteps; it++) {
                    if (!f4_wait(smem_u32(&bar_empty[s]), ph ^ 1u, 0)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&bar_full[s]);
                    mbar_arrive_expect_tx(bar, A_BYTES + B_BYTES + SA_BYTES + SB_BYTES);
                    // coordinates: x = byte along K (a multiple of 128 / of 16), y = row; rows past
                    // the end of either matrix are filled with zero bytes by the copy engine
                    const int kt = k_first + it;
                    tma_load_2d(smem_u32(smem_a + s * A_BYTES), &w_map, kt * 128, m0, bar);
                    tma_load_2d(smem_u32(smem_b + s * B_BYTES), &a_map, kt * 128, n0, bar);
                    tma_load_2d(smem_u32(smem_sa + s * SA_BYTES), &ws_map, kt * 16, m0, bar);
                    tma_load_2d(smem_u32(smem_sb + s * SB_BYTES), &as_map, kt * 16, n0, bar);
                    if (++s == ST) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // block-scaled instruction descriptor: A and B E2M1 (code 1) K-major, N = BN, scale
            // type E8M0, M = 128, scale-factor ids 0 (a block-16 MMA consumes all four bytes of a
            // column), K = 64
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) |
                                   ((uint32_t)(F4_BM >> 4) << 24);
            int s = 0, ti = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ti++) {
                // the epilogue of the tile before must have read the accumulator
                if (ti > 0 && !f4_wait(smem_u32(&bar_acc_free), (uint32_t)(ti - 1) & 1u, 5)) break;
                tcgen05_fence_after();
                for (int it = 0; it < ksteps; it++) {
                    // (the scale writers arrive only after they saw the stage's copies land)
                    if (!f4_wait(smem_u32(&bar_sf[s]), ph, 1)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_base = smem_u32(smem_a + s * A_BYTES);
                    const uint32_t b_base = smem_u32(smem_b + s * B_BYTES);
                    const uint32_t sf = tmem_sf + (uint32_t)(s * SF_COLS);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        // 64 elements of K = 32 bytes further along the swizzled 128-byte row
                        const uint64_t adesc = make_desc_sw128(a_base + kk * 32, 16, 1024);
                        const uint64_t bdesc = make_desc_sw128(b_base + kk * 32, 16, 1024);
                        tcgen05_mma_fp4_block16(tmem, adesc, bdesc, idesc, sf + (uint32_t)(kk * 4),
                                                sf + (uint32_t)(SFA_COLS + kk * NBC), (it | kk) != 0 ? 1u : 0u);
                    }
                    tcgen05_commit(smem_u32(&bar_empty[s]));
                    if (++s == ST) { s = 0; ph ^= 1u; }
                }
                tcgen05_commit(smem_u32(&bar_accum));
            }
        }
    } else {
        // ---------------- scale-factor writers ----------------
        const int q = warp & 3;                            // this warp's 32-lane quarter
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        bool ok = true;
        int s = 0, ti = 0;
        uint32_t ph = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ti++) {
        const int m0 = (tile % tiles_m) * F4_BM, n0 = (tile / tiles_m) * BN;
        for (int it = 0; it < ksteps; it++) {
            // The scale bytes travel with the stage (two more TMA boxes: 128 x 16 B and BN x 16 B),
            // so they are requested ST stages ahead like the operands.  (Loaded by the lanes
            // from global memory one stage ahead, they queued behind the operand requests in the
            // SM's request path.)  The stage's landing also means that the MMAs which read this
            // slot's tensor-memory columns a ring round ago have retired.
            if (ok) ok = f4_wait(smem_u32(&bar_full[s]), ph, 3);
            tcgen05_fence_after();
            const uint8_t* sa = smem_sa + s * SA_BYTES;
            const uint8_t* sb = smem_sb + s * SB_BYTES;
            uint4 wv[4], av[NB];
#pragma unroll
            for (int c = 0; c < 4; c++) wv[c] = *reinterpret_cast<const uint4*>(sa + (c * 32 + lane) * 16);
#pragma unroll
            for (int c = 0; c < NB; c++) av[c] = *reinterpret_cast<const uint4*>(sb + (c * 32 + lane) * 16);
            // column 4 kk + c (weights) / kk NBC + c (tokens) = word kk of row c's 16 bytes
            uint32_t wa[4][4], wb[4][NB];
#pragma unroll
            for (int c = 0; c < 4; c++) { wa[0][c] = wv[c].x; wa[1][c] = wv[c].y; wa[2][c] = wv[c].z; wa[3][c] = wv[c].w; }
#pragma unroll
            for (int c = 0; c < NB; c++) { wb[0][c] = av[c].x; wb[1][c] = av[c].y; wb[2][c] = av[c].z; wb[3][c] = av[c].w; }
            const uint32_t sf = tmem_sf + (uint32_t)(s * SF_COLS) + lane_base;
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                tcgen05_st_32x32b<4>(sf + (uint32_t)(kk * 4), wa[kk]);
                tcgen05_st_32x32b<NB>(sf + (uint32_t)(SFA_COLS + kk * NBC), wb[kk]);
            }
            tcgen05_wait_st();
            tcgen05_fence_before();
            mbar_arrive(smem_u32(&bar_sf[s]));
            if (++s == ST) { s = 0; ph ^= 1u; }
        }

        // ---------------- epilogue: tensor memory -> fp16 out[m][token] ----------------
        if (ok) ok = f4_wait(smem_u32(&bar_accum), (uint32_t)ti & 1u, 4);
        tcgen05_fence_after();
        const int m = m0 + q * 32 + lane;
        const int Z = (int)gridDim.z;
        bool reduce = false;
        if (Z > 1) {
            // Every CTA of the tile stores its fp32 partial tile; the one that finds the others'
            // already counted adds them in split order (the same sum whichever CTA comes last) and
            // writes the fp16 result.  Nobody waits for anybody.
            float* mine = part + (((size_t)tile * Z + blockIdx.z) * F4_BM + (q * 32 + lane)) * BN;
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; cb++) {
                uint32_t v[32];
                tcgen05_ld_32x32b_x32(tmem + lane_base + (uint32_t)(cb * 32), v);
                tcgen05_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    __stcg(reinterpret_cast<uint4*>(mine + cb * 32 + j), make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]));
            }
            tcgen05_fence_before();
            mbar_arrive(smem_u32(&bar_acc_free));
            __threadfence();
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            if (threadIdx.x == 64) {
                const unsigned seen = atomicAdd(counters + tile, 1u);
                s_last = (seen == (unsigned)(Z - 1));
                if (s_last) counters[tile] = 0u;                 // ready for the next launch
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            reduce = s_last != 0;
            if (reduce) __threadfence();
        }
        if (Z == 1 || reduce) {
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; cb++) {
                uint32_t v[32];
                if (Z == 1) {
                    tcgen05_ld_32x32b_x32(tmem + lane_base + (uint32_t)(cb * 32), v);
                    tcgen05_wait_ld();
                } else {
                    const float* p0 = part + (((size_t)tile * Z) * F4_BM + (q * 32 + lane)) * BN + cb * 32;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 a = __ldcg(reinterpret_cast<const float4*>(p0 + j));
                        v[j] = __float_as_uint(a.x); v[j + 1] = __float_as_uint(a.y);
                        v[j + 2] = __float_as_uint(a.z); v[j + 3] = __float_as_uint(a.w);
                    }
                    for (int z = 1; z < Z; z++) {
                        const float* pz = p0 + (size_t)z * F4_BM * BN;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(pz + j));
                            v[j] = __float_as_uint(__uint_as_float(v[j]) + a.x);
                            v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + a.y);
                            v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + a.z);
                            v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + a.w);
                        }
                    }
                }
                const int nb = n0 + cb * 32;
                if (m < M && nb < n_tokens) {
                    __half* orow = out + (size_t)m * (size_t)ld_out + nb;
                    if (nb + 32 <= n_tokens && (ld_out & 7) == 0) {
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
                            if (nb + j < n_tokens) orow[j] = __float2half(__uint_as_float(v[j]));
                    }
                }
            }
        }
        if (Z == 1) {     // this thread's part of the accumulator is read: the next tile may overwrite it
            tcgen05_fence_before();
            mbar_arrive(smem_u32(&bar_acc_free));
        }
        }   // tiles
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tcgen05_dealloc(tmem, TCOLS);
}

// ---------------------------------------------------------------------------------------------
// CTA-pair kernel (cluster of two, tcgen05 cta_group::2) for more than 128 tokens: a pair computes
// 256 weight rows x 256 tokens.  Each CTA loads its own 128 weight rows and HALF of the token tile
// (plus its rows' scale bytes and the scale bytes of all 256 tokens, which every tensor core needs);
// one thread of the pair's first CTA issues M = 256 MMAs for both SMs.  Per SM and stage that is 38
// KB from L2 instead of 54 KB - the single-CTA kernel stops at the SM's ingest rate (about 41 bytes
// per clock), not at the tensor pipe.
// Barriers (same offsets in both CTAs): full[s] local (this CTA's copies landed; its scale
// writers wait on it), sf[s] in the first CTA only (one arrival per scale-writing warp of either
// CTA once its columns are in tensor memory - which also says that CTA's operands have landed),
// empty[s] / accum committed to in each CTA.
// ---------------------------------------------------------------------------------------------
template <int ST>
__global__ void __launch_bounds__(F4_PAIR_THREADS)
gemm_fp4_pair_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap a_map,
                     const __grid_constant__ CUtensorMap ws_map, const __grid_constant__ CUtensorMap as_map,
                     __half* __restrict__ out, int M, int n_tokens, int K, int ld_out) {
    constexpr int BN = 256, HALF = 128;
    constexpr int A_BYTES = F4_BM * 128;             // this CTA's weight rows of a stage
    constexpr int B_BYTES = HALF * 128;              // this CTA's half of the token tile
    constexpr int SA_BYTES = F4_BM * 16, SB_BYTES = BN * 16;
    constexpr int NB = BN / 32;                      // token rows per lane = scale columns per MMA
    constexpr int SFA_COLS = 16, SFB_COLS = 4 * NB, SF_COLS = SFA_COLS + SFB_COLS;
    constexpr int TCOLS = f4_tmem_cols(BN + ST * SF_COLS);
    static_assert(BN + ST * SF_COLS <= 512, "tensor memory");
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + ST * A_BYTES;
    uint8_t* smem_sa = smem_b + ST * B_BYTES;
    uint8_t* smem_sb = smem_sa + ST * SA_BYTES;
    __shared__ __align__(8) uint64_t bar_full[ST];
    __shared__ __align__(8) uint64_t bar_sf[ST];
    __shared__ __align__(8) uint64_t bar_empty[ST];
    __shared__ __align__(8) uint64_t bar_accum;
    __shared__ __align__(8) uint64_t bar_acc_free;    // first CTA's: both epilogues have read the accumulators
    __shared__ uint32_t s_tmem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    // a pair walks the pair tiles pair, pair + pairs, ... (256 rows x 256 tokens each, row pair fastest)
    const int pairs = (int)(gridDim.x >> 1), pair0 = (int)(blockIdx.x >> 1);
    const int tiles_m = (M + 2 * F4_BM - 1) / (2 * F4_BM);
    const int ntiles = tiles_m * ((n_tokens + BN - 1) / BN);
    const int ksteps = K / F4_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; s++) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_sf[s]), 8);       // 4 scale-writing warps of each CTA
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_accum), 1);
        mbar_init(smem_u32(&bar_acc_free), 16);   // 8 epilogue warps of each CTA
        fence_barrier_init();
    }
    if (warp == 0) {
        tcgen05_alloc_pair(smem_u32(&s_tmem), TCOLS);
        tcgen05_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmem_sf = tmem + BN;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = pair0; tile < ntiles && ok; tile += pairs) {
                const int m0 = ((tile % tiles_m) * 2 + (int)rank) * F4_BM, n0 = (tile / tiles_m) * BN;
                const int nh = n0 + (int)rank * HALF;
                for (int it = 0; it < ksteps; it++) {
                    if (!f4_wait_poll(smem_u32(&bar_empty[s]), ph ^ 1u, 0)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&bar_full[s]);
                    mbar_arrive_expect_tx(bar, A_BYTES + B_BYTES + SA_BYTES + SB_BYTES);
                    tma_load_2d(smem_u32(smem_a + s * A_BYTES), &w_map, it * 128, m0, bar);
                    tma_load_2d(smem_u32(smem_b + s * B_BYTES), &a_map, it * 128, nh, bar);
                    tma_load_2d(smem_u32(smem_sa + s * SA_BYTES), &ws_map, it * 16, m0, bar);
                    tma_load_2d(smem_u32(smem_sb + s * SB_BYTES), &as_map, it * 16, n0, bar);
                    if (++s == ST) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) |
                                   ((uint32_t)((2 * F4_BM) >> 4) << 24);
            int s = 0, ti = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = pair0; tile < ntiles && ok; tile += pairs, ti++) {
                // both CTAs' epilogues of the tile before must have read their accumulators
                if (ti > 0 && !f4_wait_poll(smem_u32(&bar_acc_free), (uint32_t)(ti - 1) & 1u, 5)) break;
                tcgen05_fence_after();
                for (int it = 0; it < ksteps; it++) {
                    if (!f4_wait_poll(smem_u32(&bar_sf[s]), ph, 1)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_base = smem_u32(smem_a + s * A_BYTES);
                    const uint32_t b_base = smem_u32(smem_b + s * B_BYTES);
                    const uint32_t sf = tmem_sf + (uint32_t)(s * SF_COLS);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint64_t adesc = make_desc_sw128(a_base + kk * 32, 16, 1024);
                        const uint64_t bdesc = make_desc_sw128(b_base + kk * 32, 16, 1024);
                        tcgen05_mma_fp4_block16_pair(tmem, adesc, bdesc, idesc, sf + (uint32_t)(kk * 4),
                                                     sf + (uint32_t)(SFA_COLS + kk * NB), (it | kk) != 0 ? 1u : 0u);
                    }
                    const uint32_t be = smem_u32(&bar_empty[s]);
                    tcgen05_commit_pair(cluster_map_shared(be, 0));
                    tcgen05_commit_pair(cluster_map_shared(be, 1));
                    if (++s == ST) { s = 0; ph ^= 1u; }
                }
                const uint32_t ba = smem_u32(&bar_accum);
                tcgen05_commit_pair(cluster_map_shared(ba, 0));
                tcgen05_commit_pair(cluster_map_shared(ba, 1));
            }
        }
    } else {
        // ---------------- scale-factor writers (this CTA's tensor memory) ----------------
        // Two sets of four warps (a warp reaches the 32 lanes of tensor memory given by its index
        // modulo 4) take alternate stages: from the landing of a stage's bytes to the arrival on
        // sf[s] a set needs longer than the tensor core needs for the stage's MMAs.
        const int q = warp & 3;
        const int set = (warp - 2) >> 2;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        bool ok = true;
        int ti = 0;
        for (int tile = pair0; tile < ntiles; tile += pairs, ti++) {
        const int m0 = ((tile % tiles_m) * 2 + (int)rank) * F4_BM, n0 = (tile / tiles_m) * BN;
        for (int it = set; it < ksteps; it += 2) {
            const int g = ti * ksteps + it;              // stages since the kernel began
            const int s = g % ST;
            const uint32_t ph = (uint32_t)(g / ST) & 1u;
            if (ok) ok = f4_wait(smem_u32(&bar_full[s]), ph, 3);
            tcgen05_fence_after();
            const uint8_t* sa = smem_sa + s * SA_BYTES;
            const uint8_t* sb = smem_sb + s * SB_BYTES;
            uint4 wv[4], av[NB];
#pragma unroll
            for (int c = 0; c < 4; c++) wv[c] = *reinterpret_cast<const uint4*>(sa + (c * 32 + lane) * 16);
#pragma unroll
            for (int c = 0; c < NB; c++) av[c] = *reinterpret_cast<const uint4*>(sb + (c * 32 + lane) * 16);
            uint32_t wa[4][4], wb[4][NB];
#pragma unroll
            for (int c = 0; c < 4; c++) { wa[0][c] = wv[c].x; wa[1][c] = wv[c].y; wa[2][c] = wv[c].z; wa[3][c] = wv[c].w; }
#pragma unroll
            for (int c = 0; c < NB; c++) { wb[0][c] = av[c].x; wb[1][c] = av[c].y; wb[2][c] = av[c].z; wb[3][c] = av[c].w; }
            const uint32_t sf = tmem_sf + (uint32_t)(s * SF_COLS) + lane_base;
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                tcgen05_st_32x32b<4>(sf + (uint32_t)(kk * 4), wa[kk]);
                tcgen05_st_32x32b<NB>(sf + (uint32_t)(SFA_COLS + kk * NB), wb[kk]);
            }
            tcgen05_wait_st();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_map_shared(smem_u32(&bar_sf[s]), 0));
        }

        // ---------------- epilogue: this CTA's 128 rows x 256 tokens ----------------
        if (ok) ok = f4_wait_poll(smem_u32(&bar_accum), (uint32_t)ti & 1u, 4);
        tcgen05_fence_after();
        const int m = m0 + q * 32 + lane;
#pragma unroll 1
        for (int cb = set * (BN / 64); cb < (set + 1) * (BN / 64); cb++) {    // each set half of the tokens
            uint32_t v[32];
            tcgen05_ld_32x32b_x32(tmem + lane_base + (uint32_t)(cb * 32), v);
            tcgen05_wait_ld();
            const int nb = n0 + cb * 32;
            if (m < M && nb < n_tokens) {
                __half* orow = out + (size_t)m * (size_t)ld_out + nb;
                if (nb + 32 <= n_tokens && (ld_out & 7) == 0) {
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
                        if (nb + j < n_tokens) orow[j] = __float2half(__uint_as_float(v[j]));
                }
            }
        }
        // this warp's part of the accumulator is read: tell the thread that issues the next tile's MMAs
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(cluster_map_shared(smem_u32(&bar_acc_free), 0));
        }   // tiles
    }

    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 0) tcgen05_dealloc_pair(tmem, TCOLS);
}

// Workspace of the K split, one per device: fp32 partial tiles (at most F4_SPLIT_CTAS CTAs of 128 x
// 256 values) and one arrival counter per output tile (zero between launches).  Launches that split
// K share it: they must follow one another in stream order on a device.
constexpr int F4_SPLIT_CTAS = 160;
struct F4Workspace { float* part; unsigned int* counters; };
static F4Workspace g_f4_ws[NVFP4_MAX_DEVICES] = {};
static int g_f4_split = 1;          // 0: never split K
static int g_f4_persistent = 1;     // 0: one CTA per output tile
static int f4_sm_count(int dev) {
    static int sms[NVFP4_MAX_DEVICES] = {0};
    if (!sms[dev] && (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
                      sms[dev] <= 0))
        sms[dev] = 148;
    return sms[dev];
}

static bool f4_workspace(int dev, cudaStream_t st, F4Workspace* out) {
    F4Workspace& w = g_f4_ws[dev];
    if (!w.part) {
        // (an allocation is not allowed while the stream is being captured: such a launch runs unsplit)
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return false;
        float* p = nullptr;
        unsigned int* c = nullptr;
        if (cudaMalloc(&p, (size_t)F4_SPLIT_CTAS * F4_BM * 256 * sizeof(float)) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        if (cudaMalloc(&c, F4_SPLIT_CTAS * sizeof(unsigned int)) != cudaSuccess ||
            cudaMemset(c, 0, F4_SPLIT_CTAS * sizeof(unsigned int)) != cudaSuccess) {
            cudaGetLastError();
            cudaFree(p);
            if (c) cudaFree(c);
            return false;
        }
        w.part = p;
        w.counters = c;
    }
    *out = w;
    return true;
}

template <int BN, int ST>
static cudaError_t launch_fp4(const CUtensorMap& wm, const CUtensorMap& am, const CUtensorMap& ws,
                              const CUtensorMap& as, __half* out, int M, int n, int K, int ld,
                              cudaStream_t st) {
    constexpr int SMEM = ST * (F4_BM * 128 + BN * 128 + F4_BM * 16 + BN * 16) + 1024;
    static bool attr[NVFP4_MAX_DEVICES] = {false};
    const int dev = current_device_index();
    if (!attr[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_fp4_block_scaled_kernel<BN, ST>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        attr[dev] = true;
    }
    const int ntiles = ((M + F4_BM - 1) / F4_BM) * ((n + BN - 1) / BN);
    dim3 grid((unsigned)ntiles, 1, 1);
    // K split: when the output tiles leave more than half of the SMs idle AND K is deep (32 tokens
    // x 5120 rows x K 17408 is 40 tiles of 68 stages: 25.2 us unsplit, 16.3 us in three splits).
    // Meeting in the epilogue costs about 4 us, more than a 20-stage tile saves (K = 5120: 10.0 us
    // unsplit, 11.0 us split), hence the floor of 40 stages; splits keep >= 8 stages each.
    const int tiles = ntiles, total = K / F4_BK;
    int Z = 1, kper = total;
    F4Workspace w = {nullptr, nullptr};
    const int sms = f4_sm_count(dev);
    if (g_f4_split && tiles * 2 <= sms && total >= 40 && f4_workspace(dev, st, &w)) {
        Z = std::min(std::min(sms / tiles, total / 8), F4_SPLIT_CTAS / tiles);
        if (Z < 1) Z = 1;
        kper = (total + Z - 1) / Z;
        Z = (total + kper - 1) / kper;                   // no split without stages
    }
    grid.z = (unsigned)Z;
    // without a K split a CTA per SM walks the tiles (see the kernel); with one, a CTA per tile and split
    if (Z == 1 && g_f4_persistent) grid.x = (unsigned)std::min(ntiles, sms);
    gemm_fp4_block_scaled_kernel<BN, ST><<<grid, F4_THREADS, SMEM, st>>>(wm, am, ws, as, out, M, n, K, ld,
                                                                        w.part, w.counters, kper);
    return cudaGetLastError();
}

static int g_f4_pairs_override = 0;  // pairs of the tile-walking pair kernel (0: one per two SMs)
static int g_f4_pair = 1;           // the CTA-pair kernel: 1 = more than 128 tokens and K >= 10240, 2 = more than 128 tokens, 0 = never
static cudaError_t launch_fp4_pair(const CUtensorMap& wm, const CUtensorMap& am, const CUtensorMap& ws,
                                   const CUtensorMap& as, __half* out, int M, int n, int K, int ld,
                                   cudaStream_t st) {
    constexpr int ST = 5;
    constexpr int SMEM = ST * (F4_BM * 128 + 128 * 128 + F4_BM * 16 + 256 * 16) + 1024;
    static bool attr[NVFP4_MAX_DEVICES] = {false};
    const int dev = current_device_index();
    if (!attr[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_fp4_pair_kernel<ST>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        attr[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    // a pair of CTAs per pair of SMs walks the 256 x 256 tiles (one pair per tile with bit 3 of the config)
    const int ptiles = ((M + 255) / 256) * ((n + 255) / 256);
    const int pairs = g_f4_persistent ? std::min(ptiles, g_f4_pairs_override > 0 ? g_f4_pairs_override
                                                                               : f4_sm_count(dev) / 2)
                                      : ptiles;
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.blockDim = dim3(F4_PAIR_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_fp4_pair_kernel<ST>, wm, am, ws, as, out, M, n, K, ld);
}

static bool byte_matrix_map(EncodeTiledFn enc, CUtensorMap* map, const void* base, int rows, int K,
                            int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
    const cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// scale bytes [rows][K/16]: boxes of 16 bytes (one 256-element stage) x box_rows rows, unswizzled
static bool scale_matrix_map(EncodeTiledFn enc, CUtensorMap* map, const void* base, int rows, int K,
                             int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)(K / 16), (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)(K / 16)};
    const cuuint32_t box[2] = {16, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace nvfp4

extern "C" {

// out[m][t] (fp16, row pitch ld_out elements) = sum_k dequant(W)[m][k] * dequant(A)[t][k], both
// operands NVFP4 (packed [rows][K/2] + E8M0 scales [rows][K/16]).  K % 256 == 0; all five
// pointers 16-byte aligned; ld_out >= n_tokens.  0; -2 for a shape or pointer this kernel does not
// take (callers then use the W4A16 route); -3 when the driver offers no tensor-map encoder; or the
// cudaError_t of the launch.
int launch_nvfp4_gemm_fp4(const uint8_t* w_packed, const uint8_t* w_scales, const uint8_t* a_packed,
                          const uint8_t* a_scales, void* out, int M, int n_tokens, int K, int ld_out,
                          void* stream) {
    using namespace nvfp4;
    if (M <= 0 || n_tokens <= 0 || K <= 0 || K % F4_BK != 0 || ld_out < n_tokens) return NVFP4_ERR_SHAPE;
    if (!w_packed || !w_scales || !a_packed || !a_scales || !out) return NVFP4_ERR_SHAPE;
    if ((((uintptr_t)w_packed | (uintptr_t)w_scales | (uintptr_t)a_packed | (uintptr_t)a_scales |
          (uintptr_t)out) & 15) != 0)
        return NVFP4_ERR_SHAPE;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return -3;
    const int BN = n_tokens > 128 ? 256 : n_tokens > 64 ? 128 : n_tokens > 32 ? 64 : 32;
    // The pair kernel takes more than 128 tokens.  Measured at 8192 tokens: a stage costs it 790
    // cycles against 950, a tile's fixed part (prologue, cluster barriers, epilogue) 7.9 us against
    // 5.5: it wins from about 40 stages on (5120 x 17408: 310 us against 342; 6144 x 5120, 20
    // stages: 168 against 161).  Few deep-K tiles are better served by the K split.
    const int tiles1 = ((M + F4_BM - 1) / F4_BM) * ((n_tokens + 255) / 256);
    const bool few_deep = g_f4_split && tiles1 * 2 <= f4_sm_count(current_device_index()) && K / F4_BK >= 40;
    const bool pair = n_tokens > 128 && M > F4_BM && !few_deep &&
                      (g_f4_pair == 2 || (g_f4_pair == 1 && K / F4_BK >= 40));
    CUtensorMap wm, am, wsm, asm_;
    if (!byte_matrix_map(enc, &wm, w_packed, M, K, F4_BM) ||
        !byte_matrix_map(enc, &am, a_packed, n_tokens, K, pair ? 128 : BN) ||
        !scale_matrix_map(enc, &wsm, w_scales, M, K, F4_BM) ||
        !scale_matrix_map(enc, &asm_, a_scales, n_tokens, K, BN))
        return -3;
    cudaStream_t st = (cudaStream_t)stream;
    __half* o = static_cast<__half*>(out);
    const cudaError_t e =
        pair      ? launch_fp4_pair(wm, am, wsm, asm_, o, M, n_tokens, K, ld_out, st)
      : BN == 256 ? launch_fp4<256, 4>(wm, am, wsm, asm_, o, M, n_tokens, K, ld_out, st)
      : BN == 128 ? launch_fp4<128, 6>(wm, am, wsm, asm_, o, M, n_tokens, K, ld_out, st)
      : BN == 64  ? launch_fp4<64, 6>(wm, am, wsm, asm_, o, M, n_tokens, K, ld_out, st)
                  : launch_fp4<32, 6>(wm, am, wsm, asm_, o, M, n_tokens, K, ld_out, st);
    return (e == cudaSuccess) ? 0 : (int)e;
}

// 0 if no bounded wait inside the FP4 GEMM has run out since the library was loaded (or since the
// last call with reset != 0); otherwise 1 + the id of the wait.  Synchronises the device.
int nvfp4_gemm_fp4_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, nvfp4::g_fp4_status, sizeof(int)) != cudaSuccess) return -1;
    if (reset) {
        const int z = 0;
        cudaMemcpyToSymbol(nvfp4::g_fp4_status, &z, sizeof(int));
        // a launch that gave up may have left arrival counters of the K split behind
        const nvfp4::F4Workspace& w = nvfp4::g_f4_ws[nvfp4::current_device_index()];
        if (v != 0 && w.counters) cudaMemset(w.counters, 0, nvfp4::F4_SPLIT_CTAS * sizeof(unsigned int));
    }
    return v;
}

// Bit 0: K split of the FP4 GEMM for shapes with few output tiles.  Bit 1: the CTA-pair kernel for
// more than 128 tokens and K >= 10240.  Bit 2: the CTA-pair kernel for every K.  Bit 3: one CTA (pair)
// per output tile instead of one per SM (two SMs) walking the tiles.  Bits 8..15: number of pairs of
// the walking pair kernel (0 = half the SM count).  Default 3.
void nvfp4_b200_gemm_fp4_config(int flags) {
    nvfp4::g_f4_split = (flags & 1) ? 1 : 0;
    nvfp4::g_f4_pair = (flags & 4) ? 2 : (flags & 2) ? 1 : 0;
    nvfp4::g_f4_persistent = (flags & 8) ? 0 : 1;
    nvfp4::g_f4_pairs_override = (flags >> 8) & 0xFF;     // bits 8..15: CTA pairs of the tile-walking pair kernel
}

}  // extern "C"

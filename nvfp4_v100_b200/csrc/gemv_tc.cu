// NVFP4 GEMV on the block-scaled FP4 tensor-core path: y[M] = dequant(W)[M, K] . x[K], x fp16.
//
// Same entry-point semantics as the register-streaming GEMV (kernels/nvfp4_gemv.cu:38-69 kernel,
// :88-100 launcher in the reference: one fp16 activation vector, W4A16 arithmetic, fp16 output),
// with a different data path: the weight bytes and their scale bytes never pass through a
// register.  TMA streams them from HBM into a shared-memory ring and tcgen05.mma
// (kind::mxf4nvf4, 16-element E8M0 scale blocks) consumes them from there.
//
// The fp16 activation is made an FP4 operand WITHOUT rounding it: per 16-element block with
// L = 1 + floor(log2(max |x|)), each |x_k| / 2^L is a 32-bit binary fraction; its 16 base-4 digits
// d_0..d_15 (values 0..3, all exact E2M1 numbers) go to 16 token columns of the B operand, column j
// carrying the block scale 2^(L - 2j - 2) (an exact E8M0 byte).  Then sum_j (W . column_j) = W . x
// with every product exact; only the fp32 accumulation rounds.  The 16 columns are the minimum N
// of a 128-row MMA, so the digits cost no extra tensor-core time.  (Bits of an element more than
// 2^21 below its block's largest are dropped: a relative 2^-31 of that block's contribution.)
//
// Work: row tiles of 128 x K stages of 256 elements, numbered tile-major (a CTA reads consecutive
// K of the same rows: DRAM pages stay open; a K-chunk-major order measured 25 % slower); the stages
// are cut into gridDim.x equal contiguous ranges (two CTAs per SM), so a row tile's sum may span two
// or more CTAs.  Each CTA stores the partial sums of its part of a tile to a workspace slot; the
// CTA that holds the tile's last stages polls the others' slots (an empty slot holds a NaN pattern
// no sum produces; bounded wait), adds them in CTA order (deterministic) and writes the fp16
// result.  That is a wait between CTAs of one launch: the grid is at most two CTAs per SM, which
// is what fits, so all of them are resident once the previous kernel has left the SMs (a kernel
// launched behind this one cannot start before every CTA of this one runs); a CTA only waits for
// CTAs with higher indices that never wait themselves before they have stored.  If something
// else holds the SMs' shared memory for longer than the bound (about a second), the wait runs
// out, the result of that tile is wrong and nvfp4_gemv_tc_status says so; nothing hangs.
//
// One CTA (320 threads; 111 KB of shared memory: a 5-stage weight ring of 18 KB stages, an 8-slot
// ring of 2 KB digit-plane tiles, a 1 KB digit table; 256 columns of tensor memory; two CTAs per SM):
//   thread 0    TMA producer: per stage 128 rows x 128 packed bytes (128-byte swizzle) and the
//               128 x 16 scale bytes.  Two stages are requested at kernel entry, BEFORE the previous
//               kernel in the stream has finished (programmatic dependent launch: weights are
//               constants); the others once the activation loads have been issued, because those
//               would queue behind the weight requests in the SM's request path.
//   warp 1      MMA issuer (one thread): 4 x tcgen05.mma M128 N16 K64 per stage into one of two
//               accumulators.  All its stage counters are kept by increment: this thread runs one
//               instruction at a time, a division per stage would cost more than the MMAs.
//   warps 2..5  scale writers: weight scale bytes shared memory -> tensor memory (tcgen05.st; lane
//               r % 32, column r / 32, replicated in the four lane quarters) and the digit columns'
//               scale bytes, one 32-column store per stage.
//   warps 6..9  digit conversion, one 256-element stage per warp task, up to 8 stages ahead of the
//               MMAs (plane-ring slot free = the MMAs of stage i - 8 retired), with the optional
//               RMSNorm applied on the way; and the flush: accumulator (128 lanes x 16 columns)
//               -> 16-term sum per row -> slot or result, with the optional epilogue.
// Every wait is bounded; nvfp4_gemv_tc_status reports the first one that ran out.
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace nvfp4 {

constexpr int TC_BM = 128;
constexpr int TC_BK = 256;
constexpr int TC_NB = 8;                        // ring of digit-plane tiles (stages converted ahead)
constexpr int TC_THREADS = 320;
constexpr int TC_A_BYTES = TC_BM * 128;        // packed weights of a stage
constexpr int TC_B_BYTES = 16 * 128;           // activation digit planes of a stage
constexpr int TC_S_BYTES = TC_BM * 16;         // weight scale bytes of a stage
constexpr int TC_SF_COLS = 32;                 // tensor-memory columns of a stage's scale bytes
constexpr uint32_t TC_EMPTY = 0xFFFFFFFFu;      // an empty partial-sum slot
// dynamic shared memory: weight ring of st stages, digit-plane ring, digit table, exponent bytes,
// scratch; tensor memory: 2 x 16 accumulator columns + st x 32 scale columns
__host__ __device__ constexpr int tc_smem_bytes(int st) {
    return st * (TC_A_BYTES + TC_S_BYTES) + TC_NB * (TC_B_BYTES + 16) + 1024 + 128 + 1024 /*alignment*/;
}
__host__ __device__ constexpr int tc_tmem_cols(int st) { return 32 + st * TC_SF_COLS <= 128 ? 128 : 256; }

__device__ int g_tc_status = 0;

__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, int id) {
    for (uint32_t i = 0; i < (1u << 24); i++) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(20);
    }
    atomicExch(&g_tc_status, 1 + id);
    return false;
}
// the same for the two single-thread roles: plain polling
__device__ __forceinline__ bool tc_wait_poll(uint32_t bar, uint32_t parity, int id) {
    for (uint32_t i = 0; i < (1u << 26); i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(&g_tc_status, 1 + id);
    return false;
}

__device__ __forceinline__ void tc_mma(uint32_t taddr, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::
            "r"(taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ void tc_st_x4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(taddr), "r"(a),
                 "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tc_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tc_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ uint32_t tc_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// the CTA whose range [b total / G, (b + 1) total / G) holds stage g
__device__ __forceinline__ int tc_cta_of(unsigned g, unsigned total, unsigned G) {
    return (int)(((g + 1u) * G - 1u) / total);
}

// The 32-bit fraction |x| / 2^L of an fp16 bit pattern (sign stripped), L = the block's exponent.
__device__ __forceinline__ uint32_t tc_fraction(uint32_t h15, int L) {
    const uint32_t e = h15 >> 10, m = h15 & 0x3FFu;
    const uint32_t m11 = e ? (m | 0x400u) : m;
    const int sh = (int)(e ? e : 1u) + 7 - L;       // |x| = m11 * 2^(max(e,1) - 25)
    return sh >= 0 ? (m11 << sh) : (sh > -32 ? (m11 >> (-sh)) : 0u);
}

// Digit planes of 8 consecutive activations (one 16-byte vector; lane o of a warp holds elements
// 8o .. 8o+7 of a 256-element stage) -> 16 words, one per plane row of the B tile, and the block's
// exponent byte.  lut[b] holds the E2M1 codes of the four base-4 digits of byte b, one per byte
// (first digit = most significant = lowest byte).
__device__ __forceinline__ void tc_digit_planes(const uint4 xv, const uint32_t* lut, uint8_t* btile,
                                                uint8_t* lbytes, int lane) {
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
    uint32_t hmax = 0;
#pragma unroll
    for (int w = 0; w < 4; w++) {
        hmax = max(hmax, xw[w] & 0x7FFFu);
        hmax = max(hmax, (xw[w] >> 16) & 0x7FFFu);
    }
    hmax = max(hmax, __shfl_xor_sync(0xffffffffu, hmax, 1));   // lanes 2b, 2b+1 share block b
    const uint32_t em = hmax >> 10;
    const uint32_t m11 = em ? ((hmax & 0x3FFu) | 0x400u) : (hmax & 0x3FFu);
    const int L = (32 - __clz(m11)) + (int)(em ? em : 1u) - 25;
    uint32_t u[8], sgn = 0;
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const uint32_t h = (xw[e >> 1] >> (16 * (e & 1))) & 0xFFFFu;
        u[e] = tc_fraction(h & 0x7FFFu, L);
        sgn |= ((h >> 12) & 8u) << (4 * e);
    }
#pragma unroll
    for (int q = 0; q < 4; q++) {                  // planes 4q .. 4q+3 = byte 3-q of the fraction
        uint32_t pr[4];
#pragma unroll
        for (int i = 0; i < 4; i++)               // elements 2i (low nibble) and 2i+1 (high)
            pr[i] = lut[(u[2 * i] >> (24 - 8 * q)) & 0xFFu] | (lut[(u[2 * i + 1] >> (24 - 8 * q)) & 0xFFu] << 4);
        // 4x4 byte transpose: pr[i] byte p -> plane p byte i
        const uint32_t t0 = tc_prmt(pr[0], pr[1], 0x5140u), t1 = tc_prmt(pr[2], pr[3], 0x5140u);
        const uint32_t t2 = tc_prmt(pr[0], pr[1], 0x7362u), t3 = tc_prmt(pr[2], pr[3], 0x7362u);
        const uint32_t o[4] = {tc_prmt(t0, t1, 0x5410u), tc_prmt(t0, t1, 0x7632u),
                               tc_prmt(t2, t3, 0x5410u), tc_prmt(t2, t3, 0x7632u)};
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const int row = 4 * q + p;
            const int chunk = (lane >> 2) ^ (row & 7);      // 128-byte swizzle
            *reinterpret_cast<uint32_t*>(btile + row * 128 + chunk * 16 + (lane & 3) * 4) = o[p] | sgn;
        }
    }
    if ((lane & 1) == 0) lbytes[lane >> 1] = (uint8_t)(L + 125);
}

// What the kernel fuses around the dot products (the arithmetic of the register-streaming GEMV's
// prologues and epilogues, which is that of rmsnorm_kernel and silu_mul_kernel):
//   TPRO_RMSNORM: x' = f16(f32(x) * rsqrt(mean(x^2) + eps) * w1[k]) is what gets multiplied
//   TEPI_RESIDUAL: out[m] = f16(f32(residual[m]) + f32(f16(y[m])))
//   TEPI_SILU_MUL: rows in groups of 16 = 8 gate rows then 8 up rows; out[8 g + r] =
//                  f16(f32(f16(silu(f16(gate)))) * f32(f16(up)))
enum { TPRO_NONE = 0, TPRO_RMSNORM = 1 };
enum { TEPI_STORE = 0, TEPI_RESIDUAL = 1, TEPI_SILU_MUL = 2 };
struct TcFuse {
    const float* norm_w1;
    float eps;
    const __half* residual;
    int pre;       // weight stages requested at kernel entry; the others follow the activation request
};

// Final value of row `row` (this lane's; the warp's 32 rows are consecutive and start at a
// multiple of 32) -> output.
template <int EPI>
__device__ __forceinline__ void tc_store(float tot, int row, int lane, int M, __half* y, const TcFuse& fz) {
    if (EPI == TEPI_SILU_MUL) {
        const float up = __shfl_down_sync(0xffffffffu, tot, 8);     // lanes 8..15 / 24..31: up rows
        if ((lane & 8) == 0 && row + 8 < M) {
            const float gf = round_f16(tot), uf = round_f16(up);
            const float sl = round_f16(gf / (1.0f + expf(-gf)));
            y[(row >> 4) * 8 + (lane & 7)] = __float2half(sl * uf);
        }
    } else if (row < M) {
        if (EPI == TEPI_RESIDUAL) {
            const __half* res = fz.residual;
            PDL_FRESH(res);
            y[row] = __float2half(__half2float(res[row]) + round_f16(tot));
        } else {
            y[row] = __float2half(tot);
        }
    }
}

// DBG: every CTA folds the global nanosecond timer at its pipeline events into `dbg` (a timing
// probe, see nvfp4_gemv_tc_probe): word 0 = earliest kernel entry, 1 = latest entry, 2 / 3 = latest /
// earliest "previous kernel finished", 4 = latest digit planes done, 5 = latest first MMA, 6 = latest
// accumulation retired, 7 = latest flush done, 8 = latest CTA end.  Words 0 and 3 start at the
// largest int64, the others at 0.
__device__ __forceinline__ long long tc_now() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
template <int ST, int PRO, int EPI, bool DBG>
__global__ void __launch_bounds__(TC_THREADS)
gemv_tc_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap s_map,
               const __half* x, __half* y, float* part, unsigned int* counters, int M, int K,
               const TcFuse fz, long long* dbg_) {
    long long* dbg = dbg_;
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    constexpr int NB = TC_NB, TC_TMEM_COLS = tc_tmem_cols(ST);
    const bool rec = DBG;
    if (rec && threadIdx.x == 0) { const long long t = tc_now(); atomicMin(dbg + 0, t); atomicMax(dbg + 1, t); }
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~(uintptr_t)1023);
    uint8_t* smem_a = smem;                                   // ST x 16 KB packed weights
    uint8_t* smem_b = smem_a + ST * TC_A_BYTES;               // NB x 2 KB digit planes
    uint8_t* smem_s = smem_b + NB * TC_B_BYTES;               // ST x 2 KB weight scale bytes
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem_s + ST * TC_S_BYTES);   // 256 words
    uint8_t* smem_l = reinterpret_cast<uint8_t*>(lut + 256);  // NB x 16 exponent bytes
    float* s_part = reinterpret_cast<float*>(smem_l + NB * 16);              // 9 partial sums
    __shared__ __align__(8) uint64_t bar_full[ST];            // TMA bytes landed
    __shared__ __align__(8) uint64_t bar_ready[ST];           // scale bytes written to tensor memory
    __shared__ __align__(8) uint64_t bar_empty[ST];           // the stage's MMAs retired
    __shared__ __align__(8) uint64_t bar_bfull[NB];           // digit planes of a stage written
    __shared__ __align__(8) uint64_t bar_bempty[NB];          // the MMAs that read them retired
    __shared__ __align__(8) uint64_t bar_acc_full[2];         // a segment's accumulation retired
    __shared__ __align__(8) uint64_t bar_acc_empty[2];        // the flush warps have read it
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_xreq;                           // the activation loads have been issued

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, b = blockIdx.x;
    const int ntiles = (M + TC_BM - 1) / TC_BM, nk = K / TC_BK;
    // (the launcher keeps total * (G + 1) below 2^32: 32-bit divisions)
    const unsigned total = (unsigned)ntiles * (unsigned)nk;
    const unsigned g0 = (unsigned)b * total / (unsigned)G, g1 = (unsigned)(b + 1) * total / (unsigned)G;
    // the loops below count stages with 32-bit counters kept by increment: the single-thread roles
    // (copy issue, MMA issue) run one instruction at a time, a division per stage would cost them
    // more than the stage's four MMAs
    const int nst = (int)(g1 - g0);                  // stages of this CTA
    const int tile0 = (int)(g0 / nk), ks0 = (int)(g0 % nk);

    // The copy-issuing thread starts the first ST stages at once: it needs only the barriers, which
    // it initialises itself; tensor memory, the digit table and the other warps come later.
    int p_s = 0, p_tile = tile0, p_ks = ks0, p_i = 0;       // producer state (thread 0)
    uint32_t p_ph = 0;
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&w_map) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&s_map) : "memory");
        for (int s = 0; s < ST; s++) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_ready[s]), 128);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int s = 0; s < NB; s++) {
            mbar_init(smem_u32(&bar_bfull[s]), 1);
            mbar_init(smem_u32(&bar_bempty[s]), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(smem_u32(&bar_acc_full[a]), 1);
            mbar_init(smem_u32(&bar_acc_empty[a]), 128);
        }
        s_xreq = 0;
        fence_barrier_init();
        for (; p_i < nst && p_i < ST && p_i < fz.pre; p_i++) {
            const uint32_t bar = smem_u32(&bar_full[p_s]);
            mbar_arrive_expect_tx(bar, TC_A_BYTES + TC_S_BYTES);
            tma_load_2d(smem_u32(smem_a + p_s * TC_A_BYTES), &w_map, p_ks * 128, p_tile * TC_BM, bar);
            tma_load_2d(smem_u32(smem_s + p_s * TC_S_BYTES), &s_map, p_ks * 16, p_tile * TC_BM, bar);
            if (++p_s == ST) { p_s = 0; p_ph ^= 1u; }
            if (++p_ks == nk) { p_ks = 0; p_tile++; }
        }
    }
    if (warp == 1) {
        tcgen05_alloc(smem_u32(&s_tmem), TC_TMEM_COLS);
        tcgen05_relinquish();
    }
    if (threadIdx.x >= 64) {                                  // digit-code table, one entry each
        const uint32_t v = threadIdx.x - 64;
        uint32_t w = 0;
#pragma unroll
        for (int p = 0; p < 4; p++) w |= ((0x5420u >> (4 * ((v >> (6 - 2 * p)) & 3u))) & 0xFu) << (8 * p);
        lut[v] = w;
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmem_sf = tmem + 32;

    if (warp == 0) {
        // ---------------- TMA producer, the stages after the first ST ----------------
        if (lane == 0) {
            // the stages held back at entry go out once the activation loads are on their way: in
            // the SM's request path they would otherwise queue behind 90 KB of weight requests
            for (uint32_t w = 0; w < (1u << 24) && s_xreq == 0; w++) {}
            for (; p_i < nst; p_i++) {
                if (!tc_wait_poll(smem_u32(&bar_empty[p_s]), p_ph ^ 1u, 0)) break;
                const uint32_t bar = smem_u32(&bar_full[p_s]);
                mbar_arrive_expect_tx(bar, TC_A_BYTES + TC_S_BYTES);
                tma_load_2d(smem_u32(smem_a + p_s * TC_A_BYTES), &w_map, p_ks * 128, p_tile * TC_BM, bar);
                tma_load_2d(smem_u32(smem_s + p_s * TC_S_BYTES), &s_map, p_ks * 16, p_tile * TC_BM, bar);
                if (++p_s == ST) { p_s = 0; p_ph ^= 1u; }
                if (++p_ks == nk) { p_ks = 0; p_tile++; }
            }
        }
    } else {
        // converting warps: the loads of the next stage to convert are kept one conversion ahead;
        // the first stage's norm weights (constants) are requested before the previous kernel has
        // finished, its activations right after, together with the loads of the mean of squares
        int cv = 0, cv_ks = 0;
        uint4 pre_x = make_uint4(0u, 0u, 0u, 0u);
        float4 pre_w0 = make_float4(0.f, 0.f, 0.f, 0.f), pre_w1 = pre_w0;
        if (warp >= 6) {
            cv = warp - 6;
            cv_ks = ks0 + cv;
            while (cv_ks >= nk) cv_ks -= nk;
            if (PRO == TPRO_RMSNORM && cv < nst) {
                pre_w0 = __ldg(reinterpret_cast<const float4*>(fz.norm_w1 + cv_ks * TC_BK + lane * 8));
                pre_w1 = __ldg(reinterpret_cast<const float4*>(fz.norm_w1 + cv_ks * TC_BK + lane * 8 + 4));
            }
        }
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        PDL_FRESH(x);
        PDL_FRESH(y);
        PDL_FRESH(part);
        PDL_FRESH(counters);
        if (warp >= 6 && cv < nst) pre_x = *reinterpret_cast<const uint4*>(x + cv_ks * TC_BK + lane * 8);
        if (PRO != TPRO_RMSNORM && threadIdx.x == 192) s_xreq = 1;
        if (rec && threadIdx.x == 32) { const long long t = tc_now(); atomicMax(dbg + 2, t); atomicMin(dbg + 3, t); }
        float inv = 1.0f;
        if (PRO == TPRO_RMSNORM) {
            // mean of squares over the WHOLE activation (K <= 5 * 8 * 288), all loads in flight at once
            const int t0 = (int)threadIdx.x - 32;
            constexpr int T = TC_THREADS - 32;
            uint4 v[5];
#pragma unroll
            for (int j = 0; j < 5; j++) {
                const int i = (t0 + j * T) * 8;
                v[j] = (i < K) ? *reinterpret_cast<const uint4*>(x + i) : make_uint4(0u, 0u, 0u, 0u);
            }
            if (threadIdx.x == 192) s_xreq = 1;
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 5; j++) {
                const __half2* h = reinterpret_cast<const __half2*>(&v[j]);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(h[e]);
                    ss = fmaf(f.x, f.x, ss);
                    ss = fmaf(f.y, f.y, ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) s_part[warp - 1] = ss;
            asm volatile("bar.sync 1, 288;\n" ::: "memory");
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < 9; w++) tot += s_part[w];
            inv = rsqrtf(tot / (float)K + fz.eps);
        }
        if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                // A, B E2M1 K-major; N = 16; E8M0 scales; M = 128
                const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(16 >> 3) << 17) | (1u << 23) |
                                       ((uint32_t)(TC_BM >> 4) << 24);
                // descriptors: +1 in the low word = 16 bytes further in shared memory
                const uint64_t a_desc0 = make_desc_sw128(smem_u32(smem_a), 16, 1024);
                const uint64_t b_desc0 = make_desc_sw128(smem_u32(smem_b), 16, 1024);
                int s = 0, ks = ks0, seg = 0, bs = 0;
                uint32_t ph = 0;
                bool first = true;
                for (int i = 0; i < nst; i++) {
                    const int buf = seg & 1;
                    if (first &&  // the flush warps must have drained this accumulator's previous use
                        !tc_wait_poll(smem_u32(&bar_acc_empty[buf]), (((uint32_t)seg >> 1) & 1u) ^ 1u, 1))
                        break;
                    // the scale writers arrive here only after they saw the stage's copies land and
                    // its digit planes written
                    if (!tc_wait_poll(smem_u32(&bar_ready[s]), ph, 3)) break;
                    tcgen05_fence_after();
                    if (rec && i == 0) atomicMax(dbg + 5, tc_now());
                    const uint64_t adesc = a_desc0 + (uint64_t)(s * (TC_A_BYTES >> 4));
                    const uint64_t bdesc = b_desc0 + (uint64_t)(bs * (TC_B_BYTES >> 4));
                    const uint32_t sf = tmem_sf + (uint32_t)(s * TC_SF_COLS);
                    const uint32_t d = tmem + (uint32_t)(buf * 16);
                    tc_mma(d, adesc, bdesc, idesc, sf, sf + 16, first ? 0u : 1u);
                    tc_mma(d, adesc + 2, bdesc + 2, idesc, sf + 4, sf + 20, 1u);
                    tc_mma(d, adesc + 4, bdesc + 4, idesc, sf + 8, sf + 24, 1u);
                    tc_mma(d, adesc + 6, bdesc + 6, idesc, sf + 12, sf + 28, 1u);
                    tcgen05_commit(smem_u32(&bar_empty[s]));
                    tcgen05_commit(smem_u32(&bar_bempty[bs]));
                    first = false;
                    if (++s == ST) { s = 0; ph ^= 1u; }
                    bs = (bs + 1) & (NB - 1);
                    if (++ks == nk || i == nst - 1) {       // the segment ends with this stage
                        tcgen05_commit(smem_u32(&bar_acc_full[buf]));
                        seg++;
                        first = true;
                        ks = 0;
                    }
                }
            }
        } else if (warp < 6) {
            // ---------------- scale writers ----------------
            const int q = warp & 3;                               // lane quarter
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            const uint32_t sub = 0x01010101u * (uint32_t)(2 * (lane & 15));
            bool ok = true;
            int s = 0, bs = 0;
            uint32_t ph = 0, bph = 0;
            for (int i = 0; i < nst; i++) {
                if (ok) ok = tc_wait(smem_u32(&bar_bfull[bs]), bph, 6);
                // digit column n, block blk: exponent byte L_blk + 125 - 2n (word kk = blocks 4kk..)
                const uint4 lw = *reinterpret_cast<const uint4*>(smem_l + bs * 16);
                if (ok) ok = tc_wait(smem_u32(&bar_full[s]), ph, 4);
                tcgen05_fence_after();
                const uint32_t sf = tmem_sf + (uint32_t)(s * TC_SF_COLS) + lane_base;
                // weight scales: row c*32 + lane holds 16 bytes = 4 MMAs x 4 blocks
                const uint8_t* ss = smem_s + s * TC_S_BYTES;
                const uint4 r0 = *reinterpret_cast<const uint4*>(ss + (0 * 32 + lane) * 16);
                const uint4 r1 = *reinterpret_cast<const uint4*>(ss + (1 * 32 + lane) * 16);
                const uint4 r2 = *reinterpret_cast<const uint4*>(ss + (2 * 32 + lane) * 16);
                const uint4 r3 = *reinterpret_cast<const uint4*>(ss + (3 * 32 + lane) * 16);
                // one store of the stage's 32 scale columns: 16 for the weights (4 per MMA), 16 for
                // the digit columns (1 per MMA on a 4-column boundary)
                const uint32_t cols[32] = {r0.x, r1.x, r2.x, r3.x, r0.y, r1.y, r2.y, r3.y,
                                           r0.z, r1.z, r2.z, r3.z, r0.w, r1.w, r2.w, r3.w,
                                           lw.x - sub, 0u, 0u, 0u, lw.y - sub, 0u, 0u, 0u,
                                           lw.z - sub, 0u, 0u, 0u, lw.w - sub, 0u, 0u, 0u};
                tc_st_x32(sf, cols);
                tc_wait_st();
                tcgen05_fence_before();
                mbar_arrive(smem_u32(&bar_ready[s]));
                if (++s == ST) { s = 0; ph ^= 1u; }
                if (++bs == NB) { bs = 0; bph ^= 1u; }
            }
        } else {
            // ---------------- digit conversion (ahead of the MMAs) and flush ----------------
            // Warp f of the four converts the stages i = f, f + 4, ... of this CTA's range, one
            // 256-element stage (32 octets) a time, into plane-ring slot i % 8 - as far ahead as
            // the ring allows (slot free = the MMAs of stage i - 8 retired).  Before it waits for
            // a segment's accumulation it has converted its stages up to 7 beyond the segment's
            // end: those waits depend only on MMAs inside or before the segment, and the MMAs of
            // the next segment find their planes ready.
            const int q = warp & 3;
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            auto convert_upto = [&](int last) {
                for (; cv <= last && cv < nst; cv += 4) {
                    const int slot = cv & (NB - 1);
                    uint4 xv = pre_x;
                    if (PRO == TPRO_RMSNORM) {
                        const float w[8] = {pre_w0.x, pre_w0.y, pre_w0.z, pre_w0.w,
                                            pre_w1.x, pre_w1.y, pre_w1.z, pre_w1.w};
                        __half2* h = reinterpret_cast<__half2*>(&xv);
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float2 fv = __half22float2(h[e]);
                            h[e] = __halves2half2(__float2half(fv.x * inv * w[2 * e]),
                                                  __float2half(fv.y * inv * w[2 * e + 1]));
                        }
                    }
                    cv_ks += 4;
                    while (cv_ks >= nk) cv_ks -= nk;
                    if (cv + 4 < nst) {                  // the next conversion's loads travel meanwhile
                        const int k = cv_ks * TC_BK + lane * 8;
                        pre_x = *reinterpret_cast<const uint4*>(x + k);
                        if (PRO == TPRO_RMSNORM) {
                            pre_w0 = __ldg(reinterpret_cast<const float4*>(fz.norm_w1 + k));
                            pre_w1 = __ldg(reinterpret_cast<const float4*>(fz.norm_w1 + k + 4));
                        }
                    }
                    // the slot's previous planes (stage cv - 8) must have been consumed
                    tc_wait(smem_u32(&bar_bempty[slot]), (((uint32_t)cv >> 3) & 1u) ^ 1u, 7);
                    tc_digit_planes(xv, lut, smem_b + slot * TC_B_BYTES, smem_l + slot * 16, lane);
                    fence_proxy_async_smem();        // the tensor core reads the planes (async proxy)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_bfull[slot]));
                }
            };
            int seg = 0, tile = tile0, left = nst, seg_len = nk - ks0, done = 0;
            while (left > 0) {
                if (seg_len > left) seg_len = left;
                convert_upto(done + seg_len - 1 + (NB - 1));
                if (rec && seg == 0 && lane == 0) atomicMax(dbg + 4, tc_now());
                const int buf = seg & 1;
                const bool got = tc_wait(smem_u32(&bar_acc_full[buf]), ((uint32_t)seg >> 1) & 1u, 5);
                tcgen05_fence_after();
                if (rec && lane == 0) atomicMax(dbg + 6, tc_now());
                uint32_t v[16];
                tc_ld_x16(tmem + lane_base + (uint32_t)(buf * 16), v);
                tcgen05_wait_ld();
                tcgen05_fence_before();
                mbar_arrive(smem_u32(&bar_acc_empty[buf]));
                float sum = 0.0f;
#pragma unroll
                for (int j = 15; j >= 0; j--) sum += __uint_as_float(v[j]);   // small digits first
                if (!got) sum = 0.0f;
                const int row = tile * TC_BM + q * 32 + lane;
                const int c_first = tc_cta_of((unsigned)tile * nk, total, G);
                const int c_last = tc_cta_of((unsigned)(tile + 1) * nk - 1u, total, G);
                if (c_first == c_last) {
                    tc_store<EPI>(sum, row, lane, M, y, fz);
                } else if (b != c_first) {
                    // a contributor: one store into slot (tile + CTA) - unique, because a CTA
                    // boundary inside a tile adds one slot - and done.  An empty slot holds the
                    // all-ones pattern (a NaN no sum of products produces); the value IS the flag.
                    uint32_t bits = __float_as_uint(sum);
                    if (bits == TC_EMPTY) bits = 0x7FFFFFFFu;
                    __stcg(reinterpret_cast<unsigned int*>(&part[(size_t)(tile + b) * TC_BM + q * 32 + lane]), bits);
                } else {
                    // the reducer: the CTA with the tile's FIRST stages, for which this is the last
                    // segment of its range (the contributors meet the tile at the start of theirs,
                    // or lie wholly inside it and end when this CTA ends; none of them ever waits,
                    // so there is no chain of waits).  It polls their slots until none is empty
                    // (bounded), adds its own part and theirs in CTA order, and leaves the slots
                    // empty for the next launch: one memory round trip on the critical path, where
                    // fence + counter + fence + loads took four.
                    float tot = sum;
                    for (int c = c_first + 1; c <= c_last; c += 8) {     // eight loads in flight
                        uint32_t pv[8];
                        bool all = false;
                        for (uint32_t spin = 0; spin < (1u << 20) && !all; spin++) {
                            all = true;
#pragma unroll
                            for (int u = 0; u < 8; u++) {
                                pv[u] = 0u;
                                if (c + u <= c_last) {
                                    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(pv[u])
                                                 : "l"(&part[(size_t)(tile + c + u) * TC_BM + q * 32 + lane]) : "memory");
                                    all = all && (pv[u] != TC_EMPTY);
                                }
                            }
                        }
                        if (!all) atomicExch(&g_tc_status, 9);
#pragma unroll
                        for (int u = 0; u < 8; u++)
                            if (c + u <= c_last) {
                                tot += __uint_as_float(pv[u]);
                                __stcg(reinterpret_cast<unsigned int*>(&part[(size_t)(tile + c + u) * TC_BM + q * 32 + lane]),
                                       TC_EMPTY);
                            }
                    }
                    tc_store<EPI>(tot, row, lane, M, y, fz);
                }
                left -= seg_len;
                done += seg_len;
                seg_len = nk;
                tile++;
                seg++;
            }
            if (rec && lane == 0) atomicMax(dbg + 7, tc_now());
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem, TC_TMEM_COLS);
    if (rec && threadIdx.x == 32) atomicMax(dbg + 8, tc_now());
}

// ---------------------------------------------------------------------------------------------
// The MLP block of a decoder layer in ONE launch:
//   phase 0: act = silu(gate) * up,  [gate; up] = W_gu . rmsnorm(h)      (rows interleaved in 8s)
//   phase 1: h  += W_down . act
// i.e. launch_nvfp4_gemv_tc_fused(prologue 1, epilogue 2) followed by (prologue 0, epilogue 1), with
// the same arithmetic, roles and partial-sum protocol as gemv_tc_kernel.  What the fusion buys: the
// weight ring never drains between the two matrices - while the flush warps finish phase 0 and
// meet at a grid-wide barrier (all of `act` must exist before any CTA converts a stage of it), the
// producer already streams W_down into the ring slots the last gate/up stages free - and one
// kernel boundary per layer disappears.  The barrier is a counter + generation pair in global
// memory that resets itself (the generation is read after the previous kernel has finished and
// cannot change before this CTA itself has arrived); the wait is bounded.  Like the reducer's wait
// it needs every CTA of the grid resident: two per SM.
// ---------------------------------------------------------------------------------------------
struct TcMlpArgs {
    __half* h;                 // residual stream [hidden], in and out
    __half* act;               // [inter] scratch
    const float* norm_w1;      // post-attention RMSNorm weights (1 + w), fp32 [hidden]
    float eps;
    int inter, hidden;
    float* part;               // partial-sum slots: (ntiles0 + G) for phase 0, then those of phase 1
    unsigned int* gbar;        // {arrival count, generation}
    int pre;                   // weight stages requested at kernel entry
};
struct TcRange { int ntiles, nk, nst, tile0, ks0; unsigned total; };
__device__ __forceinline__ TcRange tc_range(int M, int K, unsigned G, unsigned b) {
    TcRange r;
    r.ntiles = (M + TC_BM - 1) / TC_BM;
    r.nk = K / TC_BK;
    r.total = (unsigned)r.ntiles * (unsigned)r.nk;
    const unsigned g0 = b * r.total / G, g1 = (b + 1) * r.total / G;
    r.nst = (int)(g1 - g0);
    r.tile0 = (int)(g0 / r.nk);
    r.ks0 = (int)(g0 % r.nk);
    return r;
}

template <int ST>
__global__ void __launch_bounds__(TC_THREADS)
gemv_tc_mlp_kernel(const __grid_constant__ CUtensorMap w_map0, const __grid_constant__ CUtensorMap s_map0,
                   const __grid_constant__ CUtensorMap w_map1, const __grid_constant__ CUtensorMap s_map1,
                   const TcMlpArgs a) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    constexpr int NB = TC_NB, TC_TMEM_COLS = tc_tmem_cols(ST);
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem_a + ST * TC_A_BYTES;
    uint8_t* smem_s = smem_b + NB * TC_B_BYTES;
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem_s + ST * TC_S_BYTES);
    uint8_t* smem_l = reinterpret_cast<uint8_t*>(lut + 256);
    float* s_part = reinterpret_cast<float*>(smem_l + NB * 16);
    __shared__ __align__(8) uint64_t bar_full[ST];
    __shared__ __align__(8) uint64_t bar_ready[ST];
    __shared__ __align__(8) uint64_t bar_empty[ST];
    __shared__ __align__(8) uint64_t bar_bfull[NB];
    __shared__ __align__(8) uint64_t bar_bempty[NB];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_xreq;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned G = gridDim.x, b = blockIdx.x;
    const int M0 = 2 * a.inter, K0 = a.hidden, M1 = a.hidden, K1 = a.inter;
    const TcRange R0 = tc_range(M0, K0, G, b), R1 = tc_range(M1, K1, G, b);

    int p_s = 0, p_i = 0;                                   // producer state (thread 0)
    uint32_t p_ph = 0;
    int p_tile = R0.tile0, p_ks = R0.ks0;
    auto issue0 = [&]() {
        const uint32_t bar = smem_u32(&bar_full[p_s]);
        mbar_arrive_expect_tx(bar, TC_A_BYTES + TC_S_BYTES);
        tma_load_2d(smem_u32(smem_a + p_s * TC_A_BYTES), &w_map0, p_ks * 128, p_tile * TC_BM, bar);
        tma_load_2d(smem_u32(smem_s + p_s * TC_S_BYTES), &s_map0, p_ks * 16, p_tile * TC_BM, bar);
        if (++p_s == ST) { p_s = 0; p_ph ^= 1u; }
        if (++p_ks == R0.nk) { p_ks = 0; p_tile++; }
    };
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&w_map0) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&s_map0) : "memory");
        for (int s = 0; s < ST; s++) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_ready[s]), 128);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int s = 0; s < NB; s++) {
            mbar_init(smem_u32(&bar_bfull[s]), 1);
            mbar_init(smem_u32(&bar_bempty[s]), 1);
        }
        for (int c = 0; c < 2; c++) {
            mbar_init(smem_u32(&bar_acc_full[c]), 1);
            mbar_init(smem_u32(&bar_acc_empty[c]), 128);
        }
        s_xreq = 0;
        fence_barrier_init();
        for (; p_i < R0.nst && p_i < ST && p_i < a.pre; p_i++) issue0();
    }
    if (warp == 1) {
        tcgen05_alloc(smem_u32(&s_tmem), TC_TMEM_COLS);
        tcgen05_relinquish();
    }
    if (threadIdx.x >= 64) {
        const uint32_t v = threadIdx.x - 64;
        uint32_t w = 0;
#pragma unroll
        for (int p = 0; p < 4; p++) w |= ((0x5420u >> (4 * ((v >> (6 - 2 * p)) & 3u))) & 0xFu) << (8 * p);
        lut[v] = w;
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tmem_sf = tmem + 32;

    if (warp == 0) {
        // ---------------- TMA producer: the rest of W_gu, then W_down, without a pause ----------------
        if (lane == 0) {
            for (uint32_t w = 0; w < (1u << 24) && s_xreq == 0; w++) {}
            bool ok = true;
            for (; p_i < R0.nst && ok; p_i++) {
                ok = tc_wait_poll(smem_u32(&bar_empty[p_s]), p_ph ^ 1u, 0);
                if (ok) issue0();
            }
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&w_map1) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&s_map1) : "memory");
            p_tile = R1.tile0;
            p_ks = R1.ks0;
            for (int i = 0; i < R1.nst && ok; i++) {
                // as at kernel entry: only a.pre stages of the second matrix are requested before
                // the flush warps have passed the barrier and issued their loads of `act`; the
                // tail of phase 0 (partial sums, barrier) needs the SM's request path short
                if (i == a.pre)
                    for (uint32_t w = 0; w < (1u << 24) && s_xreq < 2; w++) {}
                ok = tc_wait_poll(smem_u32(&bar_empty[p_s]), p_ph ^ 1u, 0);
                if (!ok) break;
                const uint32_t bar = smem_u32(&bar_full[p_s]);
                mbar_arrive_expect_tx(bar, TC_A_BYTES + TC_S_BYTES);
                tma_load_2d(smem_u32(smem_a + p_s * TC_A_BYTES), &w_map1, p_ks * 128, p_tile * TC_BM, bar);
                tma_load_2d(smem_u32(smem_s + p_s * TC_S_BYTES), &s_map1, p_ks * 16, p_tile * TC_BM, bar);
                if (++p_s == ST) { p_s = 0; p_ph ^= 1u; }
                if (++p_ks == R1.nk) { p_ks = 0; p_tile++; }
            }
        }
    } else {
        __half* h = a.h;
        __half* act = a.act;
        float* part = a.part;
        unsigned int* gbar = a.gbar;
        // first conversion of this warp (phase 0): norm weights before the wait, activations after
        int cv = 0, cv_ks = 0;
        uint4 pre_x = make_uint4(0u, 0u, 0u, 0u);
        float4 pre_w0 = make_float4(0.f, 0.f, 0.f, 0.f), pre_w1 = pre_w0;
        if (warp >= 6) {
            cv = warp - 6;
            cv_ks = R0.ks0 + cv;
            while (cv_ks >= R0.nk) cv_ks -= R0.nk;
            if (cv < R0.nst) {
                pre_w0 = __ldg(reinterpret_cast<const float4*>(a.norm_w1 + cv_ks * TC_BK + lane * 8));
                pre_w1 = __ldg(reinterpret_cast<const float4*>(a.norm_w1 + cv_ks * TC_BK + lane * 8 + 4));
            }
        }
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        PDL_FRESH(h);
        PDL_FRESH(act);
        PDL_FRESH(part);
        PDL_FRESH(gbar);
        if (warp >= 6 && cv < R0.nst) pre_x = *reinterpret_cast<const uint4*>(h + cv_ks * TC_BK + lane * 8);
        // generation of the grid barrier: cannot change before this CTA has arrived
        unsigned int gen0;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(gen0) : "l"(gbar + 1) : "memory");
        float inv;
        {
            const int t0 = (int)threadIdx.x - 32;
            constexpr int T = TC_THREADS - 32;
            uint4 v[5];
#pragma unroll
            for (int j = 0; j < 5; j++) {
                const int i = (t0 + j * T) * 8;
                v[j] = (i < K0) ? *reinterpret_cast<const uint4*>(h + i) : make_uint4(0u, 0u, 0u, 0u);
            }
            if (threadIdx.x == 192) s_xreq = 1;
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 5; j++) {
                const __half2* hh = reinterpret_cast<const __half2*>(&v[j]);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(hh[e]);
                    ss = fmaf(f.x, f.x, ss);
                    ss = fmaf(f.y, f.y, ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) s_part[warp - 1] = ss;
            asm volatile("bar.sync 1, 288;\n" ::: "memory");
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < 9; w++) tot += s_part[w];
            inv = rsqrtf(tot / (float)K0 + a.eps);
        }
        if (warp == 1) {
            // ---------------- MMA issuer: both phases, one stage sequence ----------------
            if (lane == 0) {
                const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(16 >> 3) << 17) | (1u << 23) |
                                       ((uint32_t)(TC_BM >> 4) << 24);
                const uint64_t a_desc0 = make_desc_sw128(smem_u32(smem_a), 16, 1024);
                const uint64_t b_desc0 = make_desc_sw128(smem_u32(smem_b), 16, 1024);
                int s = 0, seg = 0, bs = 0;
                uint32_t ph = 0;
                bool ok = true;
                for (int p = 0; p < 2 && ok; p++) {
                    const int nst = p ? R1.nst : R0.nst, nk = p ? R1.nk : R0.nk;
                    int ks = p ? R1.ks0 : R0.ks0;
                    bool first = true;
                    for (int i = 0; i < nst; i++) {
                        const int buf = seg & 1;
                        if (first &&
                            !tc_wait_poll(smem_u32(&bar_acc_empty[buf]), (((uint32_t)seg >> 1) & 1u) ^ 1u, 1)) {
                            ok = false;
                            break;
                        }
                        if (!tc_wait_poll(smem_u32(&bar_ready[s]), ph, 3)) { ok = false; break; }
                        tcgen05_fence_after();
                        const uint64_t adesc = a_desc0 + (uint64_t)(s * (TC_A_BYTES >> 4));
                        const uint64_t bdesc = b_desc0 + (uint64_t)(bs * (TC_B_BYTES >> 4));
                        const uint32_t sf = tmem_sf + (uint32_t)(s * TC_SF_COLS);
                        const uint32_t d = tmem + (uint32_t)(buf * 16);
                        tc_mma(d, adesc, bdesc, idesc, sf, sf + 16, first ? 0u : 1u);
                        tc_mma(d, adesc + 2, bdesc + 2, idesc, sf + 4, sf + 20, 1u);
                        tc_mma(d, adesc + 4, bdesc + 4, idesc, sf + 8, sf + 24, 1u);
                        tc_mma(d, adesc + 6, bdesc + 6, idesc, sf + 12, sf + 28, 1u);
                        tcgen05_commit(smem_u32(&bar_empty[s]));
                        tcgen05_commit(smem_u32(&bar_bempty[bs]));
                        first = false;
                        if (++s == ST) { s = 0; ph ^= 1u; }
                        bs = (bs + 1) & (NB - 1);
                        if (++ks == nk || i == nst - 1) {
                            tcgen05_commit(smem_u32(&bar_acc_full[buf]));
                            seg++;
                            first = true;
                            ks = 0;
                        }
                    }
                }
            }
        } else if (warp < 6) {
            // ---------------- scale writers: one sequence of nst0 + nst1 stages ----------------
            const int q = warp & 3;
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            const uint32_t sub = 0x01010101u * (uint32_t)(2 * (lane & 15));
            bool ok = true;
            int s = 0, bs = 0;
            uint32_t ph = 0, bph = 0;
            const int n_all = R0.nst + R1.nst;
            for (int i = 0; i < n_all; i++) {
                if (ok) ok = tc_wait(smem_u32(&bar_bfull[bs]), bph, 6);
                const uint4 lw = *reinterpret_cast<const uint4*>(smem_l + bs * 16);
                if (ok) ok = tc_wait(smem_u32(&bar_full[s]), ph, 4);
                tcgen05_fence_after();
                const uint32_t sf = tmem_sf + (uint32_t)(s * TC_SF_COLS) + lane_base;
                const uint8_t* ss = smem_s + s * TC_S_BYTES;
                const uint4 r0 = *reinterpret_cast<const uint4*>(ss + (0 * 32 + lane) * 16);
                const uint4 r1 = *reinterpret_cast<const uint4*>(ss + (1 * 32 + lane) * 16);
                const uint4 r2 = *reinterpret_cast<const uint4*>(ss + (2 * 32 + lane) * 16);
                const uint4 r3 = *reinterpret_cast<const uint4*>(ss + (3 * 32 + lane) * 16);
                const uint32_t cols[32] = {r0.x, r1.x, r2.x, r3.x, r0.y, r1.y, r2.y, r3.y,
                                           r0.z, r1.z, r2.z, r3.z, r0.w, r1.w, r2.w, r3.w,
                                           lw.x - sub, 0u, 0u, 0u, lw.y - sub, 0u, 0u, 0u,
                                           lw.z - sub, 0u, 0u, 0u, lw.w - sub, 0u, 0u, 0u};
                tc_st_x32(sf, cols);
                tc_wait_st();
                tcgen05_fence_before();
                mbar_arrive(smem_u32(&bar_ready[s]));
                if (++s == ST) { s = 0; ph ^= 1u; }
                if (++bs == NB) { bs = 0; bph ^= 1u; }
            }
        } else {
            // ---------------- digit conversion and flush, phase 0, barrier, phase 1 ----------------
            const int q = warp & 3;
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            int seg = 0;
            for (int p = 0; p < 2; p++) {
                const TcRange& R = p ? R1 : R0;
                const int base = p ? R0.nst : 0;             // index of the phase's first stage in the CTA's sequence
                const int M = p ? M1 : M0;
                const __half* x = p ? act : h;
                float* pslots = part + (p ? (size_t)(R0.ntiles + (int)G) * TC_BM : 0);
                TcFuse fz;
                fz.norm_w1 = a.norm_w1;
                fz.eps = a.eps;
                fz.residual = h;
                fz.pre = a.pre;
                if (p == 1) {
                    // ---- grid barrier: every CTA's part of `act` is stored ----
                    asm volatile("bar.sync 2, 128;\n" ::: "memory");
                    if (threadIdx.x == 192) {
                        __threadfence();
                        const unsigned int old = atomicAdd(gbar, 1u);
                        if (old == G - 1u) {
                            atomicExch(gbar, 0u);
                            __threadfence();
                            atomicAdd(gbar + 1, 1u);
                        }
                        bool passed = false;             // one poller per CTA
                        for (uint32_t spin = 0; spin < (1u << 22) && !passed; spin++) {
                            unsigned int g;
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(g) : "l"(gbar + 1) : "memory");
                            passed = (g != gen0);
                            if (!passed) __nanosleep(40);
                        }
                        if (!passed) atomicExch(&g_tc_status, 10);
                    }
                    asm volatile("bar.sync 2, 128;\n" ::: "memory");
                    // this warp's first stage of phase 1: sequence index = f (mod 4), at or after base
                    const int f = warp - 6;
                    cv = base + ((f - base) & 3);
                    cv_ks = R.ks0 + (cv - base);
                    while (cv_ks >= R.nk) cv_ks -= R.nk;
                    if (cv - base < R.nst)
                        pre_x = __ldcg(reinterpret_cast<const uint4*>(x + cv_ks * TC_BK + lane * 8));
                    if (threadIdx.x == 192) s_xreq = 2;
                }
                auto convert_upto = [&](int last) {            // `last`: index within the phase
                    for (; cv - base <= last && cv - base < R.nst; cv += 4) {
                        const int slot = cv & (NB - 1);
                        uint4 xv = pre_x;
                        if (p == 0) {
                            const float w[8] = {pre_w0.x, pre_w0.y, pre_w0.z, pre_w0.w,
                                                pre_w1.x, pre_w1.y, pre_w1.z, pre_w1.w};
                            __half2* hh = reinterpret_cast<__half2*>(&xv);
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const float2 fv = __half22float2(hh[e]);
                                hh[e] = __halves2half2(__float2half(fv.x * inv * w[2 * e]),
                                                       __float2half(fv.y * inv * w[2 * e + 1]));
                            }
                        }
                        cv_ks += 4;
                        while (cv_ks >= R.nk) cv_ks -= R.nk;
                        if (cv + 4 - base < R.nst) {
                            const int k = cv_ks * TC_BK + lane * 8;
                            if (p == 0) {
                                pre_x = *reinterpret_cast<const uint4*>(x + k);
                                pre_w0 = __ldg(reinterpret_cast<const float4*>(a.norm_w1 + k));
                                pre_w1 = __ldg(reinterpret_cast<const float4*>(a.norm_w1 + k + 4));
                            } else {
                                pre_x = __ldcg(reinterpret_cast<const uint4*>(x + k));
                            }
                        }
                        tc_wait(smem_u32(&bar_bempty[slot]), (((uint32_t)cv >> 3) & 1u) ^ 1u, 7);
                        tc_digit_planes(xv, lut, smem_b + slot * TC_B_BYTES, smem_l + slot * 16, lane);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bar_bfull[slot]));
                    }
                };
                int tile = R.tile0, left = R.nst, seg_len = R.nk - R.ks0, done = 0;
                while (left > 0) {
                    if (seg_len > left) seg_len = left;
                    convert_upto(done + seg_len - 1 + (NB - 1));
                    const int buf = seg & 1;
                    const bool got = tc_wait(smem_u32(&bar_acc_full[buf]), ((uint32_t)seg >> 1) & 1u, 5);
                    tcgen05_fence_after();
                    uint32_t v[16];
                    tc_ld_x16(tmem + lane_base + (uint32_t)(buf * 16), v);
                    tcgen05_wait_ld();
                    tcgen05_fence_before();
                    mbar_arrive(smem_u32(&bar_acc_empty[buf]));
                    float sum = 0.0f;
#pragma unroll
                    for (int j = 15; j >= 0; j--) sum += __uint_as_float(v[j]);
                    if (!got) sum = 0.0f;
                    const int row = tile * TC_BM + q * 32 + lane;
                    const int c_first = tc_cta_of((unsigned)tile * R.nk, R.total, G);
                    const int c_last = tc_cta_of((unsigned)(tile + 1) * R.nk - 1u, R.total, G);
                    float tot = sum;
                    bool store = true;
                    if (c_first != c_last && (int)b != c_first) {
                        uint32_t bits = __float_as_uint(sum);
                        if (bits == TC_EMPTY) bits = 0x7FFFFFFFu;
                        __stcg(reinterpret_cast<unsigned int*>(&pslots[(size_t)(tile + b) * TC_BM + q * 32 + lane]), bits);
                        store = false;
                    } else if (c_first != c_last) {
                        for (int c = c_first + 1; c <= c_last; c += 8) {
                            uint32_t pv[8];
                            bool all = false;
                            for (uint32_t spin = 0; spin < (1u << 20) && !all; spin++) {
                                all = true;
#pragma unroll
                                for (int u = 0; u < 8; u++) {
                                    pv[u] = 0u;
                                    if (c + u <= c_last) {
                                        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(pv[u])
                                                     : "l"(&pslots[(size_t)(tile + c + u) * TC_BM + q * 32 + lane]) : "memory");
                                        all = all && (pv[u] != TC_EMPTY);
                                    }
                                }
                            }
                            if (!all) atomicExch(&g_tc_status, 9);
#pragma unroll
                            for (int u = 0; u < 8; u++)
                                if (c + u <= c_last) {
                                    tot += __uint_as_float(pv[u]);
                                    __stcg(reinterpret_cast<unsigned int*>(&pslots[(size_t)(tile + c + u) * TC_BM + q * 32 + lane]),
                                           TC_EMPTY);
                                }
                        }
                    }
                    // (both calls contain warp shuffles or none: `store` is uniform over the warp)
                    if (store) {
                        if (p == 0) tc_store<TEPI_SILU_MUL>(tot, row, lane, M, act, fz);
                        else tc_store<TEPI_RESIDUAL>(tot, row, lane, M, h, fz);
                    }
                    left -= seg_len;
                    done += seg_len;
                    seg_len = R.nk;
                    tile++;
                    seg++;
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem, TC_TMEM_COLS);
}

// Per-device workspace (partial sums + counters), grown on demand outside stream capture.
struct TcWorkspace { float* part = nullptr; unsigned int* counters = nullptr; size_t slots = 0, tiles = 0; };
static TcWorkspace g_tc_ws[NVFP4_MAX_DEVICES];
static long long* g_tc_probe = nullptr;   // device buffer of 8 x 16 words while the timing probe is on
static unsigned g_tc_probe_seq = 0;       // launches since the probe was switched on

static bool tc_workspace(int dev, size_t slots, size_t tiles, TcWorkspace** out) {
    TcWorkspace& w = g_tc_ws[dev];
    if (w.slots < slots || w.tiles < tiles) {
        if (w.part) cudaFree(w.part);
        if (w.counters) cudaFree(w.counters);
        w = TcWorkspace();
        const size_t ns = slots < 4096 ? 4096 : slots, nt = tiles < 4096 ? 4096 : tiles;
        if (cudaMalloc(&w.part, ns * TC_BM * sizeof(float)) != cudaSuccess) return false;
        if (cudaMalloc(&w.counters, nt * 4 * sizeof(unsigned int)) != cudaSuccess) return false;
        if (cudaMemset(w.counters, 0, nt * 4 * sizeof(unsigned int)) != cudaSuccess) return false;
        if (cudaMemset(w.part, 0xFF, ns * TC_BM * sizeof(float)) != cudaSuccess) return false;   // all slots empty
        w.slots = ns;
        w.tiles = nt;
    }
    *out = &w;
    return true;
}

}  // namespace nvfp4

namespace nvfp4 {

template <int ST, int PRO, int EPI, bool DBG>
static cudaError_t tc_launch_st(int dev, int G, cudaStream_t st, const CUtensorMap& wm,
                                 const CUtensorMap& sm, const __half* x, __half* y, TcWorkspace* ws,
                                 int M, int K, const TcFuse& fz, long long* dbg) {
    static bool attr[NVFP4_MAX_DEVICES] = {false};      // per instantiation and device
    if (!attr[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(gemv_tc_kernel<ST, PRO, EPI, DBG>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   tc_smem_bytes(ST));
        if (e != cudaSuccess) return e;
        attr[dev] = true;
    }
    return launch_pdl(gemv_tc_kernel<ST, PRO, EPI, DBG>, dim3((unsigned)G), dim3(TC_THREADS),
                      (size_t)tc_smem_bytes(ST), st, wm, sm, x, y, ws->part, ws->counters, M, K, fz, dbg);
}
static int g_tc_ring = 5;      // weight-ring depth: 5 (110 KB per CTA) or 3 (74 KB)
static int g_tc_pre = 2;       // weight stages a CTA requests at entry (the rest after its activation loads)
static int g_tc_ctas = 2;      // CTAs of one launch per SM: 2, or 1 (the next kernel's CTA fits beside it)
template <int PRO, int EPI, bool DBG>
static cudaError_t tc_launch_one(int dev, int G, size_t, cudaStream_t st, const CUtensorMap& wm,
                                 const CUtensorMap& sm, const __half* x, __half* y, TcWorkspace* ws,
                                 int M, int K, const TcFuse& fz, long long* dbg) {
    return g_tc_ring == 3 ? tc_launch_st<3, PRO, EPI, DBG>(dev, G, st, wm, sm, x, y, ws, M, K, fz, dbg)
                          : tc_launch_st<5, PRO, EPI, DBG>(dev, G, st, wm, sm, x, y, ws, M, K, fz, dbg);
}

// 0; -2 shape / pointer not taken; -3 no tensor-map encoder or no memory; else the launch error
static int tc_launch(const uint8_t* weight_packed, const uint8_t* weight_scales, const void* activation,
                     void* output, int M, int K, int pro, const float* norm_w1, float eps, int epi,
                     const void* residual, void* stream) {
    if (M <= 0 || K <= 0 || K % TC_BK != 0) return NVFP4_ERR_SHAPE;
    if (!weight_packed || !weight_scales || !activation || !output) return NVFP4_ERR_SHAPE;
    if ((((uintptr_t)weight_packed | (uintptr_t)weight_scales | (uintptr_t)activation) & 15) != 0)
        return NVFP4_ERR_SHAPE;
    if (pro < TPRO_NONE || pro > TPRO_RMSNORM || epi < TEPI_STORE || epi > TEPI_SILU_MUL) return NVFP4_ERR_SHAPE;
    if (pro == TPRO_RMSNORM && (!norm_w1 || ((uintptr_t)norm_w1 & 15) != 0 || K > 5 * 8 * (TC_THREADS - 32)))
        return NVFP4_ERR_SHAPE;
    if (epi == TEPI_RESIDUAL && !residual) return NVFP4_ERR_SHAPE;
    if (epi == TEPI_SILU_MUL && M % 16 != 0) return NVFP4_ERR_SHAPE;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return -3;
    const int dev = current_device_index();
    static int sms[NVFP4_MAX_DEVICES] = {0};
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    const int ntiles = (M + TC_BM - 1) / TC_BM, nk = K / TC_BK;
    const long long total = (long long)ntiles * nk;
    // two CTAs per SM, equal shares of the stages
    const int slots = g_tc_ctas * sms[dev];
    const int G = (int)(total < slots ? total : slots);
    if (total * (G + 1) >= (1ll << 32)) return NVFP4_ERR_SHAPE;
    const size_t smem = 0;
    TcWorkspace* ws = nullptr;
    if (!tc_workspace(dev, (size_t)ntiles + G, (size_t)ntiles, &ws)) return -3;

    CUtensorMap wm, sm;
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
        const cuuint32_t box[2] = {128, TC_BM};
        if (enc(&wm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(weight_packed), dims, strides,
                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return -3;
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)(K / 16), (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)(K / 16)};
        const cuuint32_t box[2] = {16, TC_BM};
        if (enc(&sm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(weight_scales), dims, strides,
                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return -3;
    }
    const TcFuse fz = {norm_w1, eps, static_cast<const __half*>(residual), g_tc_pre};
    const __half* x = static_cast<const __half*>(activation);
    __half* y = static_cast<__half*>(output);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
#define TC_CASE(P, E) \
    if (pro == P && epi == E) e = tc_launch_one<P, E, false>(dev, G, smem, st, wm, sm, x, y, ws, M, K, fz, nullptr); else
    if (g_tc_probe && pro == TPRO_NONE && epi == TEPI_STORE)
        e = tc_launch_one<TPRO_NONE, TEPI_STORE, true>(dev, G, smem, st, wm, sm, x, y, ws, M, K, fz,
                                                       g_tc_probe + 16 * (g_tc_probe_seq++ % 8u));
    else
    TC_CASE(TPRO_NONE, TEPI_STORE) TC_CASE(TPRO_NONE, TEPI_RESIDUAL) TC_CASE(TPRO_NONE, TEPI_SILU_MUL)
    TC_CASE(TPRO_RMSNORM, TEPI_STORE) TC_CASE(TPRO_RMSNORM, TEPI_RESIDUAL) TC_CASE(TPRO_RMSNORM, TEPI_SILU_MUL)
        e = cudaErrorInvalidValue;
#undef TC_CASE
    return (e == cudaSuccess) ? 0 : (int)e;
}

}  // namespace nvfp4

extern "C" {

// y[M] (fp16) = dequant(W)[M, K] . x[K] (fp16) on the FP4 tensor-core path.  K % 256 == 0, packed
// and scales 16-byte aligned, x 16-byte aligned.  The first call on a device (and a call with more
// row tiles than any before) allocates a workspace and must not run inside a stream capture.
// 0; -2 shape / pointer not taken; -3 no tensor-map encoder or no memory; else the launch error.
int launch_nvfp4_gemv_tc(const uint8_t* weight_packed, const uint8_t* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream) {
    return nvfp4::tc_launch(weight_packed, weight_scales, activation, output, M, K, 0, nullptr, 0.0f, 0,
                            nullptr, stream);
}

// The MLP block of a decoder layer in one launch (gemv_tc_mlp_kernel): act = silu(gate) * up over
// W_gu . rmsnorm(h) with W_gu = [2 inter][hidden], gate / up rows interleaved in groups of 8, then
// h += W_down . act with W_down = [hidden][inter].  hidden % 256 == 0, hidden <= 11520,
// inter % 256 == 0; weights and vectors 16-byte aligned.  Same return values as
// launch_nvfp4_gemv_tc; the results are those of the two fused launches it replaces.
int launch_nvfp4_mlp_tc(const uint8_t* gu_packed, const uint8_t* gu_scales, const uint8_t* down_packed,
                        const uint8_t* down_scales, void* h, void* act, const void* norm_w1, float eps,
                        int inter, int hidden, void* stream) {
    using namespace nvfp4;
    if (inter <= 0 || hidden <= 0 || hidden % TC_BK != 0 || inter % TC_BK != 0 ||
        hidden > 5 * 8 * (TC_THREADS - 32))
        return NVFP4_ERR_SHAPE;
    if (!gu_packed || !gu_scales || !down_packed || !down_scales || !h || !act || !norm_w1) return NVFP4_ERR_SHAPE;
    if ((((uintptr_t)gu_packed | (uintptr_t)gu_scales | (uintptr_t)down_packed | (uintptr_t)down_scales |
          (uintptr_t)h | (uintptr_t)act | (uintptr_t)norm_w1) & 15) != 0)
        return NVFP4_ERR_SHAPE;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return -3;
    const int dev = current_device_index();
    static int sms[NVFP4_MAX_DEVICES] = {0};
    static bool attr[NVFP4_MAX_DEVICES] = {false};
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (!attr[dev]) {
        if (cudaFuncSetAttribute(gemv_tc_mlp_kernel<5>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tc_smem_bytes(5)) != cudaSuccess)
            return -3;
        attr[dev] = true;
    }
    const int M0 = 2 * inter, K0 = hidden, M1 = hidden, K1 = inter;
    const long long nt0 = (M0 + TC_BM - 1) / TC_BM, nt1 = (M1 + TC_BM - 1) / TC_BM;
    const long long total0 = nt0 * (K0 / TC_BK), total1 = nt1 * (K1 / TC_BK);
    long long G = 2ll * sms[dev];
    if (G > total0) G = total0;
    if (G > total1) G = total1;
    if (total0 * (G + 1) >= (1ll << 32) || total1 * (G + 1) >= (1ll << 32)) return NVFP4_ERR_SHAPE;
    TcWorkspace* ws = nullptr;
    if (!tc_workspace(dev, (size_t)(nt0 + nt1 + 2 * G), 1, &ws)) return -3;
    CUtensorMap m[4];
    const cuuint32_t estr[2] = {1, 1};
    const uint8_t* bases[4] = {gu_packed, gu_scales, down_packed, down_scales};
    const int rows[4] = {M0, M0, M1, M1}, ks[4] = {K0, K0, K1, K1};
    for (int i = 0; i < 4; i++) {
        const bool sc = (i & 1) != 0;
        const cuuint64_t inner = (cuuint64_t)(sc ? ks[i] / 16 : ks[i] / 2);
        const cuuint64_t dims[2] = {inner, (cuuint64_t)rows[i]};
        const cuuint64_t strides[1] = {inner};
        const cuuint32_t box[2] = {(cuuint32_t)(sc ? 16 : 128), TC_BM};
        if (enc(&m[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(bases[i]), dims, strides, box,
                estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                sc ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                sc ? CU_TENSOR_MAP_L2_PROMOTION_NONE : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return -3;
    }
    TcMlpArgs a;
    a.h = static_cast<__half*>(h);
    a.act = static_cast<__half*>(act);
    a.norm_w1 = static_cast<const float*>(norm_w1);
    a.eps = eps;
    a.inter = inter;
    a.hidden = hidden;
    a.part = ws->part;
    a.gbar = ws->counters;
    a.pre = g_tc_pre;
    const cudaError_t e = launch_pdl(gemv_tc_mlp_kernel<5>, dim3((unsigned)G), dim3(TC_THREADS),
                                     (size_t)tc_smem_bytes(5), (cudaStream_t)stream, m[0], m[1], m[2], m[3], a);
    return (e == cudaSuccess) ? 0 : (int)e;
}

// The same with the neighbours launch_nvfp4_gemv_fused fuses: prologue 1 = RMSNorm of the
// activation with norm_w1 (fp32 [K], 1 + weight; K <= 11520), epilogue 1 = residual add, epilogue
// 2 = silu(gate) * up over gate / up rows interleaved in groups of 8 (M = 2 x outputs).
int launch_nvfp4_gemv_tc_fused(const uint8_t* weight_packed, const uint8_t* weight_scales,
                               const void* activation, void* output, int M, int K, int prologue,
                               const void* norm_w1, float eps, int epilogue, const void* residual,
                               void* stream) {
    return nvfp4::tc_launch(weight_packed, weight_scales, activation, output, M, K, prologue,
                            static_cast<const float*>(norm_w1), eps, epilogue, residual, stream);
}

// Routing of the register-streaming entry points to this kernel: calls with M * K >= a threshold
// (in units of 2^20 elements) take it when shape and alignment allow; smaller ones keep the
// register-streaming kernel, whose fixed cost per launch is lower.  0 = never route.
//   fused entry (launch_nvfp4_gemv_fused: the decode engine's calls, activation hot in L2, other
//   kernels in between): default 35 = the MLP projections, the fused input projections and the
//   vocabulary head of the 27B decoder, and on two GPUs their shards.  A decode step measured
//   258 tok/s with 40 or 60, 251 with 25, 199 with routing off on one GPU (the 31 M-element output
//   projections stay on the register-streaming kernel); on two GPUs 281 tok/s with 30, 273 with
//   40, 244 with 60 (the 37 M-element shard of the fused q/k/v projection).
//   plain entry (launch_nvfp4_gemv_v8, timed back to back on cold activations): default 40; at
//   89 M elements this kernel takes 11.4 us against 14.7 us, at 52 M 8.2 against 8.6 us, at 44.5 M
//   (the two-GPU shards of the MLP projections) 7.4 / 7.6 against 8.4 / 8.1 us, at 31 M the
//   register-streaming kernel wins (6.0 against 6.7 us).
static long long g_tc_route_min = 35ll << 20;
static long long g_tc_route_min_plain = 40ll << 20;
void nvfp4_b200_gemv_tc_config(int min_mega_elements) {
    g_tc_route_min = min_mega_elements <= 0 ? 0 : ((long long)min_mega_elements << 20);
}
void nvfp4_b200_gemv_tc_config_plain(int min_mega_elements) {
    g_tc_route_min_plain = min_mega_elements <= 0 ? 0 : ((long long)min_mega_elements << 20);
}
int nvfp4_gemv_tc_wanted(int M, int K) {
    return g_tc_route_min > 0 && (long long)M * K >= g_tc_route_min && K % nvfp4::TC_BK == 0;
}
int nvfp4_gemv_tc_wanted_plain(int M, int K) {
    return g_tc_route_min_plain > 0 && (long long)M * K >= g_tc_route_min_plain && K % nvfp4::TC_BK == 0;
}
// Weight-ring depth of the kernel: 5 stages (default; 110 KB of shared memory per CTA, two CTAs per
// SM; a decode step measured 223 tok/s) or 3 (74 KB, room for a third CTA - of the next kernel - on
// the SM; 209 tok/s).
void nvfp4_b200_gemv_tc_ring(int stages) { nvfp4::g_tc_ring = (stages == 3) ? 3 : 5; }
// Weight stages a CTA requests at kernel entry, 1..5; the others are requested once the activation
// loads have been issued.
void nvfp4_b200_gemv_tc_prefetch(int stages_at_entry) {
    nvfp4::g_tc_pre = stages_at_entry < 1 ? 1 : stages_at_entry > 5 ? 5 : stages_at_entry;
}
// CTAs of one launch per SM: 2 (default) or 1.
void nvfp4_b200_gemv_tc_ctas(int per_sm) { nvfp4::g_tc_ctas = (per_sm == 1) ? 1 : 2; }
// Allocates this device's workspace now (the launches do it on first use, which must not happen
// inside a stream capture).  0 or -3.
int nvfp4_gemv_tc_prepare(void) {
    nvfp4::TcWorkspace* ws = nullptr;
    return nvfp4::tc_workspace(nvfp4::current_device_index(), 1, 1, &ws) ? 0 : -3;
}

// Timing probe: with a device buffer of 128 int64 words, the following launches run the build that
// records the first and last CTA's pipeline events (global timer, ns) there, launch n into words
// 16 (n % 8) ..; NULL switches it off.
void nvfp4_gemv_tc_probe(void* device_buffer) {
    nvfp4::g_tc_probe = static_cast<long long*>(device_buffer);
    nvfp4::g_tc_probe_seq = 0;
}

// 0, or 1 + the id of the first bounded wait inside the tensor-core GEMV that ran out (reset != 0
// clears it).  Synchronises the device.
int nvfp4_gemv_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, nvfp4::g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (reset) {
        const int z = 0;
        cudaMemcpyToSymbol(nvfp4::g_tc_status, &z, sizeof(int));
        // after a wait that ran out, slots may have been left filled: empty them all again
        nvfp4::TcWorkspace& w = nvfp4::g_tc_ws[nvfp4::current_device_index()];
        if (v != 0 && w.part) cudaMemset(w.part, 0xFF, w.slots * nvfp4::TC_BM * sizeof(float));
    }
    return v;
}

}  // extern "C"

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
// Work: row tiles of 128 x K stages of 256 elements, numbered tile-major; the stages are cut into
// gridDim.x equal contiguous ranges (one persistent CTA per SM), so a row tile's sum may span two
// or more CTAs.  Each CTA flushes the partial sums of a (tile, range) segment to a workspace slot;
// the warp that arrives last at a tile's counter adds the slots in CTA order (deterministic) and
// writes the fp16 result.
//
// One CTA (320 threads), one per SM:
//   all warps   prologue (after the previous kernel in the stream has finished): the digit planes
//               of every K stage this CTA will visit, into a shared-memory cache (2 KB per stage, the
//               B operand tile as the tensor core reads it: 16 rows x 128 B, 128-byte swizzle), and
//               the blocks' exponent bytes.
//   warp 0      TMA producer: per stage 128 rows x 128 packed bytes (128-byte swizzle) and the
//               128 x 16 scale bytes, into an ST-stage ring; begins BEFORE the previous kernel has
//               finished (programmatic dependent launch: weights are constants).
//   warp 1      MMA issuer: 4 x tcgen05.mma M128 N16 K64 per stage into one of two accumulators.
//   warps 2..5  scale writers: weight scale bytes shared memory -> tensor memory (tcgen05.st; lane
//               r % 32, column r / 32, replicated in the four lane quarters) and the digit columns'
//               scale bytes.
//   warps 6..9  flush: accumulator (128 lanes x 16 columns) -> 16-term sum per row -> result.
// Every wait is bounded; nvfp4_gemv_tc_status reports the first one that ran out.
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace nvfp4 {

constexpr int TC_BM = 128;
constexpr int TC_BK = 256;
constexpr int TC_NBC = 20;                     // K stages whose digit planes the cache holds
constexpr int TC_THREADS = 320;
constexpr int TC_A_BYTES = TC_BM * 128;        // packed weights of a stage
constexpr int TC_B_BYTES = 16 * 128;           // activation digit planes of a stage
constexpr int TC_S_BYTES = TC_BM * 16;         // weight scale bytes of a stage
constexpr int TC_SF_COLS = 32;                 // tensor-memory columns of a stage's scale bytes
constexpr uint32_t TC_SPIN_LIMIT = 1u << 21;   // polls, each parked by the hardware for up to 1 us
__host__ __device__ constexpr int tc_smem_bytes(int st) {
    return st * (TC_A_BYTES + TC_S_BYTES) + TC_NBC * (TC_B_BYTES + 16) + 1024 /*LUT*/ + 1024 /*align*/;
}
__host__ __device__ constexpr int tc_tmem_cols(int st) {
    return 32 + st * TC_SF_COLS <= 128 ? 128 : 32 + st * TC_SF_COLS <= 256 ? 256 : 512;
}

__device__ int g_tc_status = 0;

__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, int id) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++)
        if (mbar_try_wait_hint(bar, parity, 1000u)) return true;
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

// first stage of CTA b's range, and the CTA whose range holds stage g
__device__ __forceinline__ long long tc_start(long long b, long long total, int G) { return b * total / G; }
__device__ __forceinline__ int tc_cta_of(long long g, long long total, int G) {
    return (int)(((g + 1) * G - 1) / total);
}

// The 32-bit fraction |x| / 2^L of an fp16 bit pattern (sign stripped), L = the block's exponent.
__device__ __forceinline__ uint32_t tc_fraction(uint32_t h15, int L) {
    const uint32_t e = h15 >> 10, m = h15 & 0x3FFu;
    const uint32_t m11 = e ? (m | 0x400u) : m;
    const int sh = (int)(e ? e : 1u) + 7 - L;       // |x| = m11 * 2^(max(e,1) - 25)
    return sh >= 0 ? (m11 << sh) : (sh > -32 ? (m11 >> (-sh)) : 0u);
}

// Digit planes of 8 consecutive activations (one 16-byte load) -> 16 words, one per plane row of
// the B tile, and the block's exponent.  lut[b] holds the E2M1 codes of the four base-4 digits of
// byte b, one per byte (first digit = most significant = lowest byte).
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

// DBG: CTA 0 records clock64() at its pipeline events into `dbg` (a timing probe, see
// nvfp4_gemv_tc_probe): words 0..7 = kernel entry, set-up done, previous kernel finished, digit
// planes done, last segment's accumulation retired, flush done; then per stage i < 64 four words at
// 8 + 4 i: copy issued, bytes landed (seen by a scale writer), scale bytes written, MMAs issued.
template <int ST, bool DBG>
__global__ void __launch_bounds__(TC_THREADS)
gemv_tc_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap s_map,
               const __half* x, __half* y, float* part, unsigned int* counters, int M, int K,
               long long* dbg) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const bool rec = DBG && blockIdx.x == 0;
    if (rec && threadIdx.x == 0) dbg[0] = clock64();
    constexpr int TCOLS = tc_tmem_cols(ST);
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~(uintptr_t)1023);
    uint8_t* smem_a = smem;                                   // ST x 16 KB
    uint8_t* smem_b = smem_a + ST * TC_A_BYTES;               // TC_NBC x 2 KB digit-plane cache
    uint8_t* smem_s = smem_b + TC_NBC * TC_B_BYTES;           // ST x 2 KB weight scale bytes
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem_s + ST * TC_S_BYTES);   // 256 words
    uint8_t* smem_l = reinterpret_cast<uint8_t*>(lut + 256);  // TC_NBC x 16 exponent bytes
    __shared__ __align__(8) uint64_t bar_full[ST];            // TMA bytes landed
    __shared__ __align__(8) uint64_t bar_ready[ST];           // scale bytes written to tensor memory
    __shared__ __align__(8) uint64_t bar_empty[ST];           // the stage's MMAs retired
    __shared__ __align__(8) uint64_t bar_acc_full[2];         // a segment's accumulation retired
    __shared__ __align__(8) uint64_t bar_acc_empty[2];        // the flush warps have read it
    __shared__ uint32_t s_tmem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, b = blockIdx.x;
    const int ntiles = (M + TC_BM - 1) / TC_BM, nk = K / TC_BK;
    const long long total = (long long)ntiles * nk;
    const long long g0 = tc_start(b, total, G), g1 = tc_start(b + 1, total, G);
    // the loops below count stages with 32-bit counters kept by increment: the single-thread roles
    // (copy issue, MMA issue) run one instruction at a time, a 64-bit division per stage would
    // cost them more than the stage's four MMAs
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
        for (int a = 0; a < 2; a++) {
            mbar_init(smem_u32(&bar_acc_full[a]), 1);
            mbar_init(smem_u32(&bar_acc_empty[a]), 128);
        }
        fence_barrier_init();
        for (; p_i < nst && p_i < ST; p_i++) {
            if (rec && p_i < 64) dbg[8 + 4 * p_i] = clock64();
            const uint32_t bar = smem_u32(&bar_full[p_s]);
            mbar_arrive_expect_tx(bar, TC_A_BYTES + TC_S_BYTES);
            tma_load_2d(smem_u32(smem_a + p_s * TC_A_BYTES), &w_map, p_ks * 128, p_tile * TC_BM, bar);
            tma_load_2d(smem_u32(smem_s + p_s * TC_S_BYTES), &s_map, p_ks * 16, p_tile * TC_BM, bar);
            if (++p_s == ST) { p_s = 0; p_ph ^= 1u; }
            if (++p_ks == nk) { p_ks = 0; p_tile++; }
        }
    }
    if (warp == 1) {
        tcgen05_alloc(smem_u32(&s_tmem), TCOLS);
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
    if (rec && threadIdx.x == 0) dbg[1] = clock64();

    if (warp == 0) {
        // ---------------- TMA producer (weights are constants: no wait on the previous kernel) ----
        if (lane == 0) {
            for (; p_i < nst; p_i++) {
                if (!tc_wait_poll(smem_u32(&bar_empty[p_s]), p_ph ^ 1u, 0)) break;
                if (rec && p_i < 64) dbg[8 + 4 * p_i] = clock64();
                const uint32_t bar = smem_u32(&bar_full[p_s]);
                mbar_arrive_expect_tx(bar, TC_A_BYTES + TC_S_BYTES);
                tma_load_2d(smem_u32(smem_a + p_s * TC_A_BYTES), &w_map, p_ks * 128, p_tile * TC_BM, bar);
                tma_load_2d(smem_u32(smem_s + p_s * TC_S_BYTES), &s_map, p_ks * 16, p_tile * TC_BM, bar);
                if (++p_s == ST) { p_s = 0; p_ph ^= 1u; }
                if (++p_ks == nk) { p_ks = 0; p_tile++; }
            }
        }
        // (this warp skips the digit prologue and its barrier)
    } else {
        // ---------------- digit planes of the K stages of this CTA's range ----------------
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        PDL_FRESH(x);
        PDL_FRESH(y);
        PDL_FRESH(part);
        PDL_FRESH(counters);
        if (rec && threadIdx.x == 32) dbg[2] = clock64();
        // cache slot of a stage: its K index when the cache holds all of K, else its place in this
        // CTA's range (the launcher checked that the range then fits)
        const bool by_k = nk <= TC_NBC;
        {
            const int nplanes = nst < nk ? nst : nk;
            // at most 20 stages x 32 octets over 288 threads: three per thread, all three loads
            // in flight before the first is used
            constexpr int PER = (TC_NBC * 32 + TC_THREADS - 33) / (TC_THREADS - 32);
            uint4 xv[PER];
#pragma unroll
            for (int j = 0; j < PER; j++) {
                const int t = (int)threadIdx.x - 32 + j * (TC_THREADS - 32);
                int ks = ks0 + (t >> 5);
                if (ks >= nk) ks -= nk;
                if (t < nplanes * 32)
                    xv[j] = *reinterpret_cast<const uint4*>(x + (size_t)ks * TC_BK + (t & 31) * 8);
            }
#pragma unroll
            for (int j = 0; j < PER; j++) {
                const int t = (int)threadIdx.x - 32 + j * (TC_THREADS - 32);
                int ks = ks0 + (t >> 5);
                if (ks >= nk) ks -= nk;
                const int slot = by_k ? ks : (t >> 5);
                if (t < nplanes * 32)     // uniform over a warp: t & 31 is the lane
                    tc_digit_planes(xv[j], lut, smem_b + slot * TC_B_BYTES, smem_l + slot * 16, t & 31);
            }
            fence_proxy_async_smem();          // the tensor core reads the planes (async proxy)
            asm volatile("bar.sync 1, 288;\n" ::: "memory");
            if (rec && threadIdx.x == 32) dbg[3] = clock64();
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
                int s = 0, ks = ks0, seg = 0;
                uint32_t ph = 0;
                bool first = true;
                for (int i = 0; i < nst; i++) {
                    const int buf = seg & 1;
                    if (first &&  // the flush warps must have drained this accumulator's previous use
                        !tc_wait_poll(smem_u32(&bar_acc_empty[buf]), (((uint32_t)seg >> 1) & 1u) ^ 1u, 1))
                        break;
                    // the scale writers arrive here only after they saw the stage's copies land
                    if (!tc_wait_poll(smem_u32(&bar_ready[s]), ph, 3)) break;
                    tcgen05_fence_after();
                    if (rec && i < 64) dbg[8 + 4 * i + 3] = clock64();
                    const uint64_t adesc = a_desc0 + (uint64_t)(s * (TC_A_BYTES >> 4));
                    const uint64_t bdesc = b_desc0 + (uint64_t)((by_k ? ks : i) * (TC_B_BYTES >> 4));
                    const uint32_t sf = tmem_sf + (uint32_t)(s * TC_SF_COLS);
                    const uint32_t d = tmem + (uint32_t)(buf * 16);
                    tc_mma(d, adesc, bdesc, idesc, sf, sf + 16, first ? 0u : 1u);
                    tc_mma(d, adesc + 2, bdesc + 2, idesc, sf + 4, sf + 20, 1u);
                    tc_mma(d, adesc + 4, bdesc + 4, idesc, sf + 8, sf + 24, 1u);
                    tc_mma(d, adesc + 6, bdesc + 6, idesc, sf + 12, sf + 28, 1u);
                    tcgen05_commit(smem_u32(&bar_empty[s]));
                    first = false;
                    if (++s == ST) { s = 0; ph ^= 1u; }
                    if (++ks == nk || i == nst - 1) {       // the segment ends with this stage
                        tcgen05_commit(smem_u32(&bar_acc_full[buf]));
                        seg++;
                        first = true;
                        if (ks == nk) ks = 0;
                    }
                }
            }
        } else if (warp < 6) {
            // ---------------- scale writers ----------------
            const int q = warp & 3;                               // lane quarter
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            const uint32_t sub = 0x01010101u * (uint32_t)(2 * (lane & 15));
            bool ok = true;
            int s = 0, ks = ks0;
            uint32_t ph = 0;
            for (int i = 0; i < nst; i++) {
                // digit column n, block blk: exponent byte L_blk + 125 - 2n (word kk = blocks 4kk..)
                const uint4 lw = *reinterpret_cast<const uint4*>(smem_l + (by_k ? ks : i) * 16);
                if (ok) ok = tc_wait(smem_u32(&bar_full[s]), ph, 4);
                tcgen05_fence_after();
                if (rec && i < 64 && threadIdx.x == 64) dbg[8 + 4 * i + 1] = clock64();
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
                if (rec && i < 64 && threadIdx.x == 64) dbg[8 + 4 * i + 2] = clock64();
                mbar_arrive(smem_u32(&bar_ready[s]));
                if (++s == ST) { s = 0; ph ^= 1u; }
                if (++ks == nk) ks = 0;
            }
        } else {
            // ---------------- flush ----------------
            const int q = warp & 3;
            const uint32_t lane_base = (uint32_t)(q * 32) << 16;
            int seg = 0;
            int tile = tile0, left = nst, seg_len = nk - ks0;   // stages of this tile in the range
            while (left > 0) {
                if (seg_len > left) seg_len = left;
                const int buf = seg & 1;
                const bool got = tc_wait(smem_u32(&bar_acc_full[buf]), ((uint32_t)seg >> 1) & 1u, 5);
                tcgen05_fence_after();
                if (rec && threadIdx.x == 192) dbg[4] = clock64();
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
                const int c_first = tc_cta_of((long long)tile * nk, total, G);
                const int c_last = tc_cta_of((long long)(tile + 1) * nk - 1, total, G);
                if (c_first == c_last) {
                    if (row < M) y[row] = __float2half(sum);
                } else {
                    // slot (tile + CTA) is unique: a CTA boundary inside a tile adds one slot
                    part[(size_t)(tile + b) * TC_BM + q * 32 + lane] = sum;
                    __threadfence();
                    unsigned int old = 0;
                    if (lane == 0) old = atomicAdd(&counters[tile * 4 + q], 1u);
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if (old == (unsigned int)(c_last - c_first)) {
                        __threadfence();
                        float tot = 0.0f;
                        for (int c = c_first; c <= c_last; c += 4) {   // four loads in flight
                            float pv[4];
#pragma unroll
                            for (int u = 0; u < 4; u++)
                                pv[u] = (c + u <= c_last)
                                            ? __ldcg(&part[(size_t)(tile + c + u) * TC_BM + q * 32 + lane]) : 0.0f;
#pragma unroll
                            for (int u = 0; u < 4; u++) tot += pv[u];
                        }
                        if (row < M) y[row] = __float2half(tot);
                        if (lane == 0) counters[tile * 4 + q] = 0u;   // ready for the next launch
                    }
                }
                left -= seg_len;
                seg_len = nk;
                tile++;
                seg++;
            }
            if (rec && threadIdx.x == 192) dbg[5] = clock64();
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem, TCOLS);
}

// Per-device workspace (partial sums + counters), grown on demand outside stream capture.
struct TcWorkspace { float* part = nullptr; unsigned int* counters = nullptr; size_t slots = 0, tiles = 0; };
static TcWorkspace g_tc_ws[NVFP4_MAX_DEVICES];
static int g_tc_stages = 3;     // ring depth: 3 (two CTAs per SM, the default) or 8 (one)
static long long* g_tc_probe = nullptr;   // device buffer of 264 words while the timing probe is on

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
        w.slots = ns;
        w.tiles = nt;
    }
    *out = &w;
    return true;
}

}  // namespace nvfp4

extern "C" {

// y[M] (fp16) = dequant(W)[M, K] . x[K] (fp16) on the FP4 tensor-core path.  K % 256 == 0, packed
// and scales 16-byte aligned, x 16-byte aligned.  The first call on a device (and a call with more
// row tiles than any before) allocates a workspace and must not run inside a stream capture.
// 0; -2 shape / pointer not taken; -3 no tensor-map encoder or no memory; else the launch error.
int launch_nvfp4_gemv_tc(const uint8_t* weight_packed, const uint8_t* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream) {
    using namespace nvfp4;
    if (M <= 0 || K <= 0 || K % TC_BK != 0) return NVFP4_ERR_SHAPE;
    if (!weight_packed || !weight_scales || !activation || !output) return NVFP4_ERR_SHAPE;
    if ((((uintptr_t)weight_packed | (uintptr_t)weight_scales | (uintptr_t)activation) & 15) != 0)
        return NVFP4_ERR_SHAPE;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return -3;
    const int dev = current_device_index();
    static int sms[NVFP4_MAX_DEVICES] = {0};
    static bool attr[NVFP4_MAX_DEVICES] = {false};
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (!attr[dev]) {
        if (cudaFuncSetAttribute(gemv_tc_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tc_smem_bytes(8)) != cudaSuccess ||
            cudaFuncSetAttribute(gemv_tc_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tc_smem_bytes(3)) != cudaSuccess ||
            cudaFuncSetAttribute(gemv_tc_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tc_smem_bytes(3)) != cudaSuccess)
            return -3;
        attr[dev] = true;
    }
    const int ntiles = (M + TC_BM - 1) / TC_BM, nk = K / TC_BK;
    const long long total = (long long)ntiles * nk;
    const int slots = sms[dev] * (g_tc_stages == 8 ? 1 : 2);   // resident CTAs: one or two per SM
    const int G = (int)(total < slots ? total : slots);
    // the digit-plane cache must hold every K stage a CTA visits
    const long long per_cta = (total + G - 1) / G;
    if (nk > TC_NBC && per_cta > TC_NBC) return NVFP4_ERR_SHAPE;
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
    const cudaError_t e =
        g_tc_probe
            ? launch_pdl(gemv_tc_kernel<3, true>, dim3((unsigned)G), dim3(TC_THREADS),
                         (size_t)tc_smem_bytes(3), (cudaStream_t)stream, wm, sm,
                         static_cast<const __half*>(activation), static_cast<__half*>(output), ws->part,
                         ws->counters, M, K, g_tc_probe)
        : g_tc_stages == 8
            ? launch_pdl(gemv_tc_kernel<8, false>, dim3((unsigned)G), dim3(TC_THREADS),
                         (size_t)tc_smem_bytes(8), (cudaStream_t)stream, wm, sm,
                         static_cast<const __half*>(activation), static_cast<__half*>(output), ws->part,
                         ws->counters, M, K, (long long*)nullptr)
            : launch_pdl(gemv_tc_kernel<3, false>, dim3((unsigned)G), dim3(TC_THREADS),
                         (size_t)tc_smem_bytes(3), (cudaStream_t)stream, wm, sm,
                         static_cast<const __half*>(activation), static_cast<__half*>(output), ws->part,
                         ws->counters, M, K, (long long*)nullptr);
    return (e == cudaSuccess) ? 0 : (int)e;
}

// Tuning hook: ring depth of the tensor-core GEMV: 3 stages of 18 KB and two CTAs per SM (default),
// or 8 stages and one CTA per SM.
void nvfp4_b200_gemv_tc_config(int stages) { nvfp4::g_tc_stages = (stages == 8) ? 8 : 3; }

// Timing probe: with a device buffer of 264 int64 words, the following launches run the build that
// records CTA 0's pipeline events (SM clock cycles) there; NULL switches it off.
void nvfp4_gemv_tc_probe(void* device_buffer) { nvfp4::g_tc_probe = static_cast<long long*>(device_buffer); }

// 0, or 1 + the id of the first bounded wait inside the tensor-core GEMV that ran out (reset != 0
// clears it).  Synchronises the device.
int nvfp4_gemv_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, nvfp4::g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (reset) {
        const int z = 0;
        cudaMemcpyToSymbol(nvfp4::g_tc_status, &z, sizeof(int));
    }
    return v;
}

}  // extern "C"

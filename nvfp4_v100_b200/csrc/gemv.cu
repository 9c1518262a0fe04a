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

// byte q (0..3) of w as an E8M0 scale in fp32: isolate the byte where it sits, then move it to
// the exponent field.  For q < 3 the move is an integer multiply (issued on the FMA pipe, which
// this kernel leaves almost idle) instead of a shift on the busier ALU pipe.
__device__ __forceinline__ float scale_byte(uint32_t w, int q) {
    if (q == 3) return __uint_as_float((w >> 1) & 0x7F800000u);
    return __uint_as_float((w & (0xFFu << (8 * q))) * (1u << (23 - 8 * q)));
}

// 16-byte activation load executed only where pred != 0; other lanes keep what the registers
// held (zero, set once), so no per-step zero fill is needed.
__device__ __forceinline__ void ld_x_pred(const void* p, uint32_t pred, uint32_t& r0, uint32_t& r1,
                                          uint32_t& r2, uint32_t& r3) {
    asm("{\n"
        ".reg .pred p;\n"
        "setp.ne.u32 p, %4, 0;\n"
        "@p ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%5];\n"
        "}\n"
        : "+r"(r0), "+r"(r1), "+r"(r2), "+r"(r3)
        : "r"(pred), "l"(p));
}

// Programmatic dependent launch: let the next kernel in the stream begin its weight prefetch
// while this one drains, and wait for the previous kernel before touching anything it may have
// written.  Both are no-ops when the kernel was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// Ask the L2 to fetch [p, p + bytes): both 16-byte multiples.  A prefetch has no register result,
// so it is safe on memory another kernel may still be writing: L2 is the coherence point.
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(p), "r"(bytes) : "memory");
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

    // ---- prologue that does not depend on the previous kernel: L2 prefetch of the first tile ----
    pdl_launch_dependents();
    if (blockIdx.x < ntiles) {
        const int r0 = blockIdx.x * 16;
        const int nrows = min(16, M - r0);
        // the tile's rows are adjacent in memory: one packed slab and one scale slab
        const uint8_t* pslab = packed + (size_t)r0 * prow;
        const size_t pbytes = (size_t)nrows * prow;             // multiple of 64
        const uint32_t PF_CHUNK = 8192;
        for (size_t off = (size_t)threadIdx.x * PF_CHUNK; off < pbytes;
             off += (size_t)blockDim.x * PF_CHUNK) {
            const size_t n = pbytes - off;
            prefetch_l2_bulk(pslab + off, (uint32_t)(n < PF_CHUNK ? n : PF_CHUNK));
        }
        if (threadIdx.x == blockDim.x - 1) {
            const size_t sbytes = ((size_t)nrows * srow) & ~(size_t)15;
            if (sbytes) prefetch_l2_bulk(scales + (size_t)r0 * srow, (uint32_t)sbytes);
        }
    }
    pdl_wait();

    uint32_t xr[2][8];  // two passes of activation registers (zero where this lane supplies none)
#pragma unroll
    for (int i = 0; i < 8; i++) { xr[0][i] = 0u; xr[1][i] = 0u; }

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

            // activation of this lane's chunk, 16 halves per pass (suppliers only)
            const int kc = s * 256 + t * 64;
            const uint32_t xp = (supplies && kc < K) ? 1u : 0u;
            const __half* xptr = xsrc + min(kc, K - 64);
            auto load_x = [&](int q, uint32_t (&x)[8]) {
                ld_x_pred(xptr + 16 * q, xp, x[0], x[1], x[2], x[3]);
                ld_x_pred(xptr + 16 * q + 8, xp, x[4], x[5], x[6], x[7]);
            };
            load_x(0, xr[0]);
#pragma unroll
            for (int q = 0; q < 4; q++) {  // scale block q of every chunk
                if (q < 3) load_x(q + 1, xr[(q + 1) & 1]);
                const uint32_t(&x)[8] = xr[q & 1];
                float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                    e2m1x8_to_half2x4(cur.wa[2 * q + h], a0, a1, a2, a3);
                    e2m1x8_to_half2x4(cur.wb[2 * q + h], b0, b1, b2, b3);
                    mma_f16_16816(c, a0, b0, a1, b1, x[4 * h + 0], x[4 * h + 1]);
                    mma_f16_16816(c, a2, b2, a3, b3, x[4 * h + 2], x[4 * h + 3]);
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

// ---------------------------------------------------------------------------------------------
// Same arithmetic, but the weight and scale bytes travel global -> shared with asynchronous
// copies (cp.async) into a per-thread ring of STAGES slots, so the number of bytes in flight per
// SM is set by shared memory (tens of KB per CTA) instead of by registers, and the prefetch runs
// across tile boundaries.  Every thread copies and later reads only its own slots, so the only
// synchronisation is cp.async.wait_group; slot addresses are (slot * THREADS + tid) * 16 and are
// therefore bank-conflict free.  A copy whose source lies past the end of a row is issued with a
// source size of 0, which zero-fills the slot.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, uint32_t src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_8(void* smem_dst, const void* gsrc, uint32_t src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(d), "l"(gsrc),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

template <int WARPS, int NACT, int STAGES>
__global__ void __launch_bounds__(WARPS * 32)
gemv_mma_async_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                      const __half* __restrict__ act0, const __half* __restrict__ act1,
                      __half* __restrict__ out, int M, int K) {
    constexpr int T = WARPS * 32;
    extern __shared__ __align__(16) uint8_t ring[];
    uint4* wbuf = reinterpret_cast<uint4*>(ring);                          // [STAGES][4][T]
    uint2* sbuf = reinterpret_cast<uint2*>(ring + (size_t)STAGES * 4 * T * 16);  // [STAGES][2][T]
    __shared__ float red[WARPS][16][2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nsteps = (K + 255) >> 8;
    const int ntiles = (M + 15) >> 4;
    const size_t prow = (size_t)(K >> 1), srow = (size_t)(K >> 4);
    const bool supplies = ((g & 3) == t) && (g < 4 || NACT == 2);
    const __half* xsrc = (g < 4 || NACT == 1) ? act0 : act1;

    pdl_launch_dependents();
    if (blockIdx.x < ntiles) {
        const int r0 = blockIdx.x * 16;
        const int nrows = min(16, M - r0);
        const uint8_t* pslab = packed + (size_t)r0 * prow;
        const size_t pbytes = (size_t)nrows * prow;
        const uint32_t PF_CHUNK = 8192;
        for (size_t off = (size_t)tid * PF_CHUNK; off < pbytes; off += (size_t)T * PF_CHUNK) {
            const size_t n = pbytes - off;
            prefetch_l2_bulk(pslab + off, (uint32_t)(n < PF_CHUNK ? n : PF_CHUNK));
        }
        if (tid == T - 1) {
            const size_t sbytes = ((size_t)nrows * srow) & ~(size_t)15;
            if (sbytes) prefetch_l2_bulk(scales + (size_t)r0 * srow, (uint32_t)sbytes);
        }
    }
    pdl_wait();

    // per-warp work sequence: for each of this CTA's tiles, nsw steps (step = warp + k * WARPS;
    // steps past the end of the row are issued as zero fills so every warp runs the same count)
    const int nsw = (nsteps + WARPS - 1) / WARPS;
    const int my_tiles = (blockIdx.x < ntiles) ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int total = my_tiles * nsw;

    // issue the copies of sequence element (tile index j, step index k) into ring slot `slot`
    auto issue = [&](int j, int k, int slot) {
        const int tile = blockIdx.x + j * gridDim.x;
        const int s = warp + k * WARPS;
        const int ra = min(tile * 16 + g, M - 1);
        const int rb = min(tile * 16 + g + 8, M - 1);
        const int kc = s * 256 + t * 64;            // first weight of this lane's chunk
        const bool wv = kc < K;
        const size_t poff = (size_t)(wv ? kc : 0) >> 1;
        const uint8_t* pa = packed + (size_t)ra * prow + poff;
        const uint8_t* pb = packed + (size_t)rb * prow + poff;
        const uint32_t wn = wv ? 16u : 0u;
        cp_async_16(&wbuf[(slot * 4 + 0) * T + tid], pa, wn);
        cp_async_16(&wbuf[(slot * 4 + 1) * T + tid], pa + 16, wn);
        cp_async_16(&wbuf[(slot * 4 + 2) * T + tid], pb, wn);
        cp_async_16(&wbuf[(slot * 4 + 3) * T + tid], pb + 16, wn);
        const int kg = s * 256 + (t & 1) * 128;     // first weight of this lane's scale group
        const bool sv = kg < K;
        const size_t soff = (size_t)(sv ? kg : 0) >> 4;
        cp_async_8(&sbuf[(slot * 2 + 0) * T + tid], scales + (size_t)ra * srow + soff, sv ? 8u : 0u);
        cp_async_8(&sbuf[(slot * 2 + 1) * T + tid], scales + (size_t)rb * srow + soff, sv ? 8u : 0u);
    };

    // prologue: STAGES - 1 elements in flight
    int ij = 0, ik = 0;  // (tile index, step index) of the next element to issue
#pragma unroll
    for (int p = 0; p < STAGES - 1; p++) {
        if (ij < my_tiles) issue(ij, ik, p);
        cp_async_commit();
        if (++ik == nsw) { ik = 0; ++ij; }
    }

    uint32_t xr[2][8];
#pragma unroll
    for (int i = 0; i < 8; i++) { xr[0][i] = 0u; xr[1][i] = 0u; }

    float acc_a = 0.0f, acc_b = 0.0f;
    int cj = 0, ck = 0;  // element being consumed
    for (int e = 0; e < total; e++) {
        const int slot = e % STAGES;
        // keep the ring full: the slot freed by element e-1 receives element e + STAGES - 1
        if (ij < my_tiles) issue(ij, ik, (e + STAGES - 1) % STAGES);
        cp_async_commit();
        if (++ik == nsw) { ik = 0; ++ij; }
        cp_async_wait<STAGES - 1>();  // element e has landed (this thread's own copies)

        uint32_t wa[8], wb[8];
        {
            const uint4 v0 = wbuf[(slot * 4 + 0) * T + tid], v1 = wbuf[(slot * 4 + 1) * T + tid];
            const uint4 v2 = wbuf[(slot * 4 + 2) * T + tid], v3 = wbuf[(slot * 4 + 3) * T + tid];
            wa[0] = v0.x; wa[1] = v0.y; wa[2] = v0.z; wa[3] = v0.w;
            wa[4] = v1.x; wa[5] = v1.y; wa[6] = v1.z; wa[7] = v1.w;
            wb[0] = v2.x; wb[1] = v2.y; wb[2] = v2.z; wb[3] = v2.w;
            wb[4] = v3.x; wb[5] = v3.y; wb[6] = v3.z; wb[7] = v3.w;
        }
        const uint2 sca = sbuf[(slot * 2 + 0) * T + tid], scb = sbuf[(slot * 2 + 1) * T + tid];

        const int s = warp + ck * WARPS;
        const int kc = s * 256 + t * 64;
        const uint32_t xp = (supplies && kc < K) ? 1u : 0u;
        const __half* xptr = xsrc + min(kc, K - 64);
        auto load_x = [&](int q, uint32_t (&x)[8]) {
            ld_x_pred(xptr + 16 * q, xp, x[0], x[1], x[2], x[3]);
            ld_x_pred(xptr + 16 * q + 8, xp, x[4], x[5], x[6], x[7]);
        };
        load_x(0, xr[0]);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            if (q < 3) load_x(q + 1, xr[(q + 1) & 1]);
            const uint32_t(&x)[8] = xr[q & 1];
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                e2m1x8_to_half2x4(wa[2 * q + h], a0, a1, a2, a3);
                e2m1x8_to_half2x4(wb[2 * q + h], b0, b1, b2, b3);
                mma_f16_16816(c, a0, b0, a1, b1, x[4 * h + 0], x[4 * h + 1]);
                mma_f16_16816(c, a2, b2, a3, b3, x[4 * h + 2], x[4 * h + 3]);
            }
            acc_a = fmaf(c[0], scale_byte(sca.x, q), acc_a);
            acc_a = fmaf(c[1], scale_byte(sca.y, q), acc_a);
            acc_b = fmaf(c[2], scale_byte(scb.x, q), acc_b);
            acc_b = fmaf(c[3], scale_byte(scb.y, q), acc_b);
        }

        if (++ck == nsw) {  // tile finished: combine the warps' partial sums
            const int tile = blockIdx.x + cj * gridDim.x;
            acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
            acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
            if ((t & 1) == 0) {
                red[warp][g][t >> 1] = acc_a;
                red[warp][g + 8][t >> 1] = acc_b;
            }
            __syncthreads();
            if (tid < 16 * NACT) {
                const int r = tid & 15, a = tid >> 4;
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < WARPS; w++) v += red[w][r][a];
                const int row = tile * 16 + r;
                if (row < M) out[(size_t)a * M + row] = __float2half(v);
            }
            __syncthreads();
            acc_a = 0.0f;
            acc_b = 0.0f;
            ck = 0;
            ++cj;
        }
    }
    cp_async_wait<0>();
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
    int no_pdl = 0;        // 1 = plain stream-ordered launches (no programmatic dependent launch)
    int async_ring = 0;    // 0 = register-prefetch kernel; 3, 4 or 6 = cp.async ring with that many slots
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_cfg.no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemv_mma_kernel<WARPS, NACT>, (const uint8_t*)packed,
                              (const uint8_t*)scales, (const __half*)a0, (const __half*)a1,
                              (__half*)out, M, K);
}

template <int WARPS, int NACT, int STAGES>
static cudaError_t launch_mma_async(const void* packed, const void* scales, const void* a0,
                                    const void* a1, void* out, int M, int K, cudaStream_t st) {
    constexpr int T = WARPS * 32;
    constexpr int SMEM = STAGES * T * (64 + 16);
    static int occ = 0;
    if (occ == 0) {
        if (cudaFuncSetAttribute(gemv_mma_async_kernel<WARPS, NACT, STAGES>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return cudaErrorInvalidValue;
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                &n, gemv_mma_async_kernel<WARPS, NACT, STAGES>, T, SMEM) != cudaSuccess || n <= 0)
            n = 2;
        occ = n;
    }
    const int per_sm = g_cfg.ctas_per_sm > 0 ? g_cfg.ctas_per_sm : occ;
    const int ntiles = (M + 15) / 16;
    int grid = num_sms() * per_sm;
    if (grid > ntiles) grid = ntiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(T);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_cfg.no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemv_mma_async_kernel<WARPS, NACT, STAGES>,
                              (const uint8_t*)packed, (const uint8_t*)scales, (const __half*)a0,
                              (const __half*)a1, (__half*)out, M, K);
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
        // few row tiles or a long K: spread each tile's K range over 8 warps; many tiles: 4 warps
        // per CTA and more resident CTAs (measured on B200 over the 27B layer shapes)
        if (warps == 0) warps = (K >= 8192 || (M + 15) / 16 <= 3 * num_sms()) ? 8 : 4;
        if (g_cfg.async_ring) {
            const int st_n = g_cfg.async_ring;
            if (nact == 1) {
                if (warps == 8)
                    e = (st_n == 3) ? launch_mma_async<8, 1, 3>(packed, scales, a0, a1, out, M, K, st)
                      : (st_n == 6) ? launch_mma_async<8, 1, 6>(packed, scales, a0, a1, out, M, K, st)
                                    : launch_mma_async<8, 1, 4>(packed, scales, a0, a1, out, M, K, st);
                else
                    e = (st_n == 3) ? launch_mma_async<4, 1, 3>(packed, scales, a0, a1, out, M, K, st)
                      : (st_n == 6) ? launch_mma_async<4, 1, 6>(packed, scales, a0, a1, out, M, K, st)
                                    : launch_mma_async<4, 1, 4>(packed, scales, a0, a1, out, M, K, st);
            } else {
                e = (warps == 8) ? launch_mma_async<8, 2, 4>(packed, scales, a0, a1, out, M, K, st)
                                 : launch_mma_async<4, 2, 4>(packed, scales, a0, a1, out, M, K, st);
            }
        } else if (nact == 1) {
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
// per SM used to size the grid (0 = occupancy calculator); flags bit 0 routes every call to the
// non-tensor-core kernel, bit 1 turns programmatic dependent launch off.  Returns 0, or -2 for
// an unsupported value.
int nvfp4_b200_gemv_config(int warps, int ctas_per_sm, int flags) {
    if (!(warps == 0 || warps == 2 || warps == 4 || warps == 8) || ctas_per_sm < 0)
        return NVFP4_ERR_SHAPE;
    nvfp4::g_cfg.warps = warps;
    nvfp4::g_cfg.ctas_per_sm = ctas_per_sm;
    nvfp4::g_cfg.force_generic = flags & 1;
    nvfp4::g_cfg.no_pdl = (flags >> 1) & 1;
    {
        const int ring = (flags >> 4) & 0xF;  // bits 4..7: cp.async ring slots (0, 3, 4 or 6)
        if (!(ring == 0 || ring == 3 || ring == 4 || ring == 6)) return NVFP4_ERR_SHAPE;
        nvfp4::g_cfg.async_ring = ring;
    }
    return NVFP4_OK;
}

}  // extern "C"

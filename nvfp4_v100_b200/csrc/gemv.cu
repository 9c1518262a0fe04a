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
#include "comm_layout.cuh"
#include "gemv_stream.cuh"

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

// Thread-block cluster helpers: the CTAs of a cluster split one row tile's K range and combine
// their partial sums through distributed shared memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// read a float at the same shared-memory offset as `local` in CTA `rank` of this cluster
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
    const uint32_t la = (uint32_t)__cvta_generic_to_shared(local);
    uint32_t ra;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(ra) : "r"(la), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(ra) : "memory");
    return v;
}

struct WeightRegs {
    uint32_t wa[8];  // 32 packed bytes of row g
    uint32_t wb[8];  // 32 packed bytes of row g+8
    uint2 sa, sb;    // 8 scale bytes of row g / g+8: .x = blocks 0..3 of the even chunk, .y = odd
};

// Optional work fused around the dot products (used by the decode engine; the reference-named
// entry points run with PRO_NONE / EPI_STORE).
enum { PRO_NONE = 0, PRO_RMSNORM = 1, PRO_INTERLEAVED = 2, PRO_AR_RMSNORM = 3 };
#define PRO_NV 5  // 16-byte activation vectors a thread holds in the RMSNorm prologue
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU_MUL = 2, EPI_ALLREDUCE = 3 };
struct GemvExtra {
    const float* norm_w1;     // PRO_RMSNORM: fp32 (1 + weight) [K]
    float eps;                // PRO_RMSNORM
    const __half* residual;   // EPI_RESIDUAL: fp16 [M], out = f16(residual + f16(y))
    // EPI_ALLREDUCE: every rank's communication buffer as mapped in this process, this rank,
    // the number of ranks, the data slot, and the buffers' vector capacity
    unsigned char* comm[8];
    int rank, world, parity, comm_n;
    // PRO_AR_RMSNORM: device step counter and this call's place among the n_sites all-reduces of
    // a step; sequence number of the exchange = *epoch * n_sites + site + 1
    const unsigned int* epoch;
    int site, n_sites;
};

// Layout of the push area of a communication buffer (shared with comm.cu, which owns the
// buffer): u32 push sequence at byte 16, u32 finished-CTA counter at byte 20, u32 flags[2][8] at
// byte 128, and after the pull area (256 + 4 n bytes) fp16 data[2][8][n].
#define NVFP4_PUSH_SEQ_OFF 16
#define NVFP4_PUSH_DONE_OFF 20
#define NVFP4_PUSH_FLAGS_OFF 128
#define NVFP4_PUSH_SPIN_LIMIT (1u << 22)
__device__ __forceinline__ size_t push_data_off(int n, int parity, int src) {
    return 256 + (size_t)4 * n + ((size_t)(parity * 8 + src) * n) * sizeof(__half);
}

__device__ __forceinline__ void lds_x_pred(uint32_t saddr, uint32_t pred, uint32_t& r0,
                                           uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm("{\n"
        ".reg .pred p;\n"
        "setp.ne.u32 p, %4, 0;\n"
        "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%5];\n"
        "}\n"
        : "+r"(r0), "+r"(r1), "+r"(r2), "+r"(r3)
        : "r"(pred), "r"(saddr));
}

// Tensor-core GEMV.  Requirements checked by the launcher: K % 128 == 0, packed 32-byte aligned,
// scales 8-byte aligned, activations 16-byte aligned.
//   PRO_RMSNORM : the activation is RMS-normalised first, x' = f16(f32(x) * rsqrt(mean(x^2)+eps)
//                 * w1) — the arithmetic of rmsnorm_kernel — once per CTA into shared memory
//                 (dynamic, 2K bytes), and the dot products read x' from there.
//   PRO_INTERLEAVED: (two activations) act0 holds K pairs (a0[k], a1[k]); the CTA splits them
//                 into two planes of shared memory (dynamic, 4K bytes) and reads x from there.
//   EPI_RESIDUAL: out[m] = f16(f32(residual[m]) + f32(f16(y[m]))).
//   EPI_SILU_MUL: W holds gate and up rows interleaved in groups of 8 (tile rows 0..7 = gate rows
//                 8j..8j+7, rows 8..15 = up rows 8j..8j+7; M = 2 * outputs);
//                 out[8j+r] = f16( f32(f16(silu(f16(g)))) * f32(f16(u)) ), the silu_mul_kernel chain.
//   EPI_ALLREDUCE: tensor-parallel K-split layer, GEMV and all-reduce in ONE kernel.  Every CTA
//                 stores its tile's 16 partial outputs straight into the communication buffer of
//                 EVERY rank (peer stores over NVLink, overlapping the remaining tiles' math).
//                 The CTA that finishes last on this GPU publishes "rank r, vector seq complete"
//                 to all peers, waits (bounded) for theirs, and then does
//                 out[m] = f16(f32(out[m]) + f32(f16(sum over ranks, fp32, rank order))) for the
//                 whole vector: `out` is the residual stream, updated in place.
template <int WARPS, int NACT, int PRO, int EPI>
__global__ void __launch_bounds__(WARPS * 32, 768 / (WARPS * 32))  // 24 warps per SM resident
gemv_mma_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                const __half* __restrict__ act0, const __half* __restrict__ act1,
                __half* __restrict__ out, int M, int K, GemvExtra ex) {
    __shared__ float red[WARPS][16][2];
    __shared__ float part[2][16][2];  // this CTA's partial row sums, double-buffered by tile parity
    extern __shared__ __align__(16) __half xs[];  // PRO_RMSNORM: normalised activation [K]
    // A cluster of S CTAs shares each row tile: CTA `crank` takes the K steps
    // crank*WARPS + warp (mod S*WARPS).  S = 1 when launched without a cluster.
    const int S = (int)cluster_nctarank(), crank = (int)cluster_ctarank();
    const int cid = (int)blockIdx.x / S, ncl = (int)gridDim.x / S;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gwarp = crank * WARPS + warp, gstride = S * WARPS;
    const int g = lane >> 2, t = lane & 3;
    const int nsteps = (K + 255) >> 8;
    const int ntiles = (M + 15) >> 4;
    const size_t prow = (size_t)(K >> 1), srow = (size_t)(K >> 4);
    // Lane (g,t) supplies column g of B with the activation of K chunk t when (g & 3) == t.
    const bool supplies = ((g & 3) == t) && (g < 4 || NACT == 2);
    const __half* xsrc = (g < 4 || NACT == 1) ? act0 : act1;   // re-derived after the wait below

    // ---- prologue that does not depend on the previous kernel: L2 prefetch of the first tile ----
    pdl_launch_dependents();
    if (cid < ntiles) {
        const int r0 = cid * 16;
        const int nrows = min(16, M - r0);
        // the tile's rows are adjacent in memory: one packed slab and one scale slab; the CTAs of
        // the cluster prefetch interleaved chunks of it
        const uint8_t* pslab = packed + (size_t)r0 * prow;
        const size_t pbytes = (size_t)nrows * prow;             // multiple of 64
        const uint32_t PF_CHUNK = 8192;
        for (size_t off = ((size_t)threadIdx.x * S + crank) * PF_CHUNK; off < pbytes;
             off += (size_t)blockDim.x * S * PF_CHUNK) {
            const size_t n = pbytes - off;
            prefetch_l2_bulk(pslab + off, (uint32_t)(n < PF_CHUNK ? n : PF_CHUNK));
        }
        if (threadIdx.x == blockDim.x - 1 && crank == 0) {
            const size_t sbytes = ((size_t)nrows * srow) & ~(size_t)15;
            if (sbytes) prefetch_l2_bulk(scales + (size_t)r0 * srow, (uint32_t)sbytes);
        }
    }
    // Per-warp work sequence: for each of this CTA's row tiles, nsw K steps (step = warp + k *
    // WARPS; a step past the end of the row loads nothing and contributes zero, so every warp
    // runs the same count and meets the others at each tile's reduction).  The register prefetch
    // of the next element runs across tile boundaries, so the memory pipeline drains only once
    // per CTA, not once per tile.
    const int nsw = (nsteps + gstride - 1) / gstride;
    const int my_tiles = (cid < ntiles) ? (ntiles - cid + ncl - 1) / ncl : 0;

    // row pointers of the tile the load stream is in (it runs one element ahead of the compute)
    const uint8_t *lpa, *lpb, *lsa, *lsb;
    auto set_load_tile = [&](int j) {
        const int tile = cid + j * ncl;
        const int ra = min(tile * 16 + g, M - 1);
        const int rb = min(tile * 16 + g + 8, M - 1);
        lpa = packed + (size_t)ra * prow + t * 32;
        lpb = packed + (size_t)rb * prow + t * 32;
        lsa = scales + (size_t)ra * srow + (t & 1) * 8;
        lsb = scales + (size_t)rb * srow + (t & 1) * 8;
    };
    auto load_w = [&](int k, WeightRegs& w) {
        const int s = gwarp + k * gstride;
        if (s * 256 + t * 64 < K) {
            ld_stream_256(lpa + (size_t)s * 128, w.wa);
            ld_stream_256(lpb + (size_t)s * 128, w.wb);
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) { w.wa[i] = 0u; w.wb[i] = 0u; }
        }
        if (s * 256 + (t & 1) * 128 < K) {
            w.sa = __ldg(reinterpret_cast<const uint2*>(lsa + (size_t)s * 16));
            w.sb = __ldg(reinterpret_cast<const uint2*>(lsb + (size_t)s * 16));
        } else {
            w.sa = make_uint2(0u, 0u);
            w.sb = make_uint2(0u, 0u);
        }
    };

    // The first weight loads are issued before waiting for the previous kernel: weights are never
    // written by a kernel of the step, so only the activation reads have to come after the wait.
    WeightRegs cur;
    if (my_tiles > 0) {
        set_load_tile(0);
        load_w(0, cur);  // in flight while the previous kernel drains and the activation is prepared
    }
    pdl_wait();
    // The activation loads in the main loop are plain (non-volatile) asm statements, which the
    // compiler is free to move above the wait; taking their base pointer through an asm statement
    // that is ordered after the wait pins them behind it.
    asm volatile("" : "+l"(xsrc));
    PDL_FRESH(act0); PDL_FRESH(out);
    {
        const __half* res = ex.residual;    // the residual stream is the previous kernels' output
        PDL_FRESH(res);
        ex.residual = res;
    }

    if (PRO == PRO_AR_RMSNORM) {
        // Tensor-parallel: act0 is the residual stream h, still missing the sum over the ranks of
        // the previous K-split layer's partial vectors (each rank's sits in data slot `parity`
        // of its communication buffer, written by the previous kernel).  The first few CTAs
        // (as many as it takes to cover h with one 16-byte vector per thread) do the exchange:
        // CTA 0 announces this rank's vector to the peers, each of those CTAs waits (bounded)
        // for the peers' announcements, pulls its slice of their vectors over NVLink (all peers'
        // loads in flight together: one round trip), adds the sum to h and counts itself in; the
        // last of them publishes the sequence number, which every CTA waits for (bounded) before
        // it reads h.  The weight loads above
        // are already in flight, so the exchange hides behind them.
        unsigned char* mine = ex.comm[ex.rank];
        const long long tail = nvfp4_comm_tail_offset(ex.comm_n);
        uint32_t* errw = reinterpret_cast<uint32_t*>(mine) + 1;
        uint32_t* ready = reinterpret_cast<uint32_t*>(mine + tail + NVFP4_TAIL_AR_READY_OFF);
        const uint32_t seq = *reinterpret_cast<const volatile unsigned int*>(ex.epoch) *
                                 (uint32_t)ex.n_sites + (uint32_t)ex.site + 1u;
        const int tid = threadIdx.x;
        constexpr int T = WARPS * 32;
        const int n_ar = min((int)gridDim.x, (K / 8 + T - 1) / T);    // CTAs that do the exchange
        if ((int)blockIdx.x < n_ar) {
            __shared__ int s_bad;
            if (tid == 0) s_bad = 0;
            __syncthreads();
            if (tid < ex.world && tid != ex.rank) {
                if (blockIdx.x == 0) {
                    __threadfence_system();   // this rank's partial vector (previous kernel) first
                    uint32_t* pf = reinterpret_cast<uint32_t*>(ex.comm[tid] + tail +
                                                               NVFP4_TAIL_AR_FLAGS_OFF) + ex.rank;
                    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(pf), "r"(seq) : "memory");
                }
                const uint32_t* mf = reinterpret_cast<const uint32_t*>(mine + tail +
                                                                       NVFP4_TAIL_AR_FLAGS_OFF) + tid;
                uint32_t spins = 0, v;
                do {
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(mf) : "memory");
                    if ((int32_t)(v - seq) >= 0) break;
                } while (++spins <= NVFP4_PUSH_SPIN_LIMIT);
                if ((int32_t)(v - seq) < 0) {
                    atomicExch(errw, 201u + (uint32_t)tid);
                    s_bad = 1;
                }
            }
            __syncthreads();
            if (!s_bad) {    // a missing peer's slot holds stale bytes: leave h as it is
                __half* h = const_cast<__half*>(act0);
                const size_t slot = NVFP4_COMM_DATA_OFF + (size_t)ex.parity * (size_t)ex.comm_n * 2;
                for (int i = ((int)blockIdx.x * T + tid) * 8; i < K; i += n_ar * T * 8) {
                    uint4 v[8];
#pragma unroll
                    for (int r = 0; r < 8; r++) {
                        if (r < ex.world) {
                            const void* src = ex.comm[r] + slot + (size_t)i * 2;
                            asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                         : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w)
                                         : "l"(src) : "memory");
                        }
                    }
                    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int r = 0; r < 8; r++) {
                        if (r < ex.world) {
                            const __half2* hp = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const float2 f = __half22float2(hp[e]);
                                acc[2 * e] += f.x;
                                acc[2 * e + 1] += f.y;
                            }
                        }
                    }
                    uint4 hv = *reinterpret_cast<const uint4*>(h + i);
                    __half2* hp = reinterpret_cast<__half2*>(&hv);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 f = __half22float2(hp[e]);
                        hp[e] = __floats2half2_rn(f.x + round_f16(acc[2 * e]),
                                                  f.y + round_f16(acc[2 * e + 1]));
                    }
                    *reinterpret_cast<uint4*>(h + i) = hv;
                }
            }
            // this CTA's writes to h, then its count: the barrier orders the other threads'
            // stores before thread 0's release
            __syncthreads();
            if (tid == 0) {
                // the last of the n_ar CTAs to get here publishes the sequence number
                uint32_t* done = reinterpret_cast<uint32_t*>(mine + tail + NVFP4_TAIL_AR_DONE_OFF);
                uint32_t old;
                asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;\n"
                             : "=r"(old) : "l"(done) : "memory");
                if (old == (uint32_t)n_ar - 1u) {
                    *done = 0u;
                    asm volatile("st.release.gpu.global.u32 [%0], %1;\n" ::"l"(ready), "r"(seq) : "memory");
                }
            }
        }
        if (tid == 0) {
            uint32_t spins = 0, v;
            do {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(ready) : "memory");
                if ((int32_t)(v - seq) >= 0) break;
                __nanosleep(64);
            } while (++spins <= NVFP4_PUSH_SPIN_LIMIT);
            if ((int32_t)(v - seq) < 0) atomicExch(errw, 299u);
        }
        __syncthreads();
    }
    if (PRO == PRO_RMSNORM || PRO == PRO_AR_RMSNORM) {
        // Every thread keeps its share of x in registers between the two phases and issues all
        // of its loads up front: the prologue sits on the kernel's critical path, so it must
        // cost one memory round trip, not one per loop iteration.  K <= PRO_NV * 8 * threads.
        __shared__ float s_part[WARPS];
        __shared__ float s_inv;
        constexpr int T = WARPS * 32;
        uint4 xv[PRO_NV];
#pragma unroll
        for (int j = 0; j < PRO_NV; j++) {
            const int i = (threadIdx.x + j * T) * 8;
            if (i >= K) {
                xv[j] = make_uint4(0u, 0u, 0u, 0u);
            } else if (PRO == PRO_AR_RMSNORM) {
                // h was just rewritten by CTA 0 of this very kernel: a coherent load, never the
                // read-only path
                asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(xv[j].x), "=r"(xv[j].y), "=r"(xv[j].z), "=r"(xv[j].w)
                             : "l"(act0 + i) : "memory");
            } else {
                xv[j] = *reinterpret_cast<const uint4*>(act0 + i);
            }
        }
        float4 wv[PRO_NV][2];
#pragma unroll
        for (int j = 0; j < PRO_NV; j++) {
            const int i = (threadIdx.x + j * T) * 8;
            if (i < K) {
                wv[j][0] = __ldg(reinterpret_cast<const float4*>(ex.norm_w1 + i));
                wv[j][1] = __ldg(reinterpret_cast<const float4*>(ex.norm_w1 + i + 4));
            }
        }
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < PRO_NV; j++) {
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
        if (threadIdx.x == 0) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) v += s_part[w];
            s_inv = rsqrtf(v / (float)K + ex.eps);
        }
        __syncthreads();
        const float inv = s_inv;
#pragma unroll
        for (int j = 0; j < PRO_NV; j++) {
            const int i = (threadIdx.x + j * T) * 8;
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
                *reinterpret_cast<uint4*>(xs + i) = o;
            }
        }
        __syncthreads();
    }
    if (PRO == PRO_INTERLEAVED) {
        const uint32_t* ai = reinterpret_cast<const uint32_t*>(act0);  // one u32 = (a0[k], a1[k])
        for (int i = threadIdx.x * 4; i < K; i += WARPS * 32 * 4) {
            const uint4 v = *reinterpret_cast<const uint4*>(ai + i);
            uint2 p0, p1;
            p0.x = __byte_perm(v.x, v.y, 0x5410);
            p0.y = __byte_perm(v.z, v.w, 0x5410);
            p1.x = __byte_perm(v.x, v.y, 0x7632);
            p1.y = __byte_perm(v.z, v.w, 0x7632);
            *reinterpret_cast<uint2*>(xs + i) = p0;
            *reinterpret_cast<uint2*>(xs + K + i) = p1;
        }
        __syncthreads();
    }
    uint32_t xs_base = (uint32_t)__cvta_generic_to_shared(xs) +
                       ((PRO == PRO_INTERLEAVED && g >= 4) ? (uint32_t)K * 2u : 0u);
    asm volatile("" : "+r"(xs_base));   // same for the shared-memory reads and the barrier above

    uint32_t xr[2][8];  // two passes of activation registers (zero where this lane supplies none)
#pragma unroll
    for (int i = 0; i < 8; i++) { xr[0][i] = 0u; xr[1][i] = 0u; }

    float acc_a = 0.0f, acc_b = 0.0f;
    int lj = 0, lk = 0;  // (tile index, step index) of the newest element requested from memory
    int cj = 0, ck = 0;  // (tile index, step index) of the element being computed

    // One element: request the next element into `nxt`, compute the one held in `cur`, and at a
    // tile's last step combine the warps' partial sums and write the tile's outputs.  The main
    // loop calls it with the two register buffers swapped on alternate elements, so no buffer is
    // ever copied.
    auto do_elem = [&](WeightRegs& cur, WeightRegs& nxt) {
        if (++lk == nsw) {
            lk = 0;
            if (++lj < my_tiles) set_load_tile(lj);
        }
        if (lj < my_tiles) load_w(lk, nxt);

        // activation of this lane's chunk, 16 halves per pass (suppliers only)
        const int s = gwarp + ck * gstride;
        const int kc = s * 256 + t * 64;
        const uint32_t xp = (supplies && kc < K) ? 1u : 0u;
        const int kx = max(0, min(kc, K - 64));
        const __half* xptr = xsrc + kx;
        auto load_x = [&](int q, uint32_t (&x)[8]) {
            if (PRO != PRO_NONE) {
                const uint32_t a = xs_base + (uint32_t)(kx + 16 * q) * 2u;
                lds_x_pred(a, xp, x[0], x[1], x[2], x[3]);
                lds_x_pred(a + 16u, xp, x[4], x[5], x[6], x[7]);
            } else {
                ld_x_pred(xptr + 16 * q, xp, x[0], x[1], x[2], x[3]);
                ld_x_pred(xptr + 16 * q + 8, xp, x[4], x[5], x[6], x[7]);
            }
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
        if (++ck < nsw) return;

        // ---- end of a row tile ----
        ck = 0;
        const int j = cj++;
        const int tile = cid + j * ncl;
        // lanes t=0,1 hold activation 0 (columns 0..3), lanes t=2,3 activation 1 (columns 4..7)
        acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
        acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
        if ((t & 1) == 0) {
            red[warp][g][t >> 1] = acc_a;
            red[warp][g + 8][t >> 1] = acc_b;
        }
        acc_a = 0.0f;
        acc_b = 0.0f;
        __syncthreads();
        float (*pt)[2] = part[j & 1];
        if (threadIdx.x < 32) {   // row r = tid & 15, activation a = tid >> 4
            const int r = threadIdx.x & 15, a = threadIdx.x >> 4;
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) v += red[w][r][a];
            pt[r][a] = v;
        }
        if (S > 1) cluster_sync_all();   // every CTA's partial sums are visible cluster-wide
        else __syncthreads();
        if (crank == 0) {
            if (EPI == EPI_SILU_MUL) {
                if (threadIdx.x < 8) {
                    const int r = threadIdx.x;
                    float gsum = pt[r][0], usum = pt[r + 8][0];
                    for (int c = 1; c < S; c++) {
                        gsum += ld_cluster_f32(&pt[r][0], c);
                        usum += ld_cluster_f32(&pt[r + 8][0], c);
                    }
                    if (tile * 16 + r + 8 < M) {
                        const float gf = round_f16(gsum), uf = round_f16(usum);
                        const float sl = round_f16(gf / (1.0f + expf(-gf)));
                        out[tile * 8 + r] = __float2half(sl * uf);
                    }
                }
            } else if (EPI == EPI_ALLREDUCE) {
                if ((int)threadIdx.x < ex.world) {
                    // 16 partial outputs of this tile -> slot [parity][this rank] of rank tid
                    uint4 v[2];
                    __half2* hp = reinterpret_cast<__half2*>(v);
#pragma unroll
                    for (int r = 0; r < 8; r++)
                        hp[r] = __floats2half2_rn(pt[2 * r][0], pt[2 * r + 1][0]);
                    unsigned char* dst = ex.comm[threadIdx.x] +
                                         push_data_off(ex.comm_n, ex.parity, ex.rank) +
                                         (size_t)tile * 16 * sizeof(__half);
                    reinterpret_cast<uint4*>(dst)[0] = v[0];
                    reinterpret_cast<uint4*>(dst)[1] = v[1];
                }
            } else if (threadIdx.x < 16 * NACT) {
                const int r = threadIdx.x & 15, a = threadIdx.x >> 4;
                float v = pt[r][a];
                for (int c = 1; c < S; c++) v += ld_cluster_f32(&pt[r][a], c);
                const int row = tile * 16 + r;
                if (row < M) {
                    if (EPI == EPI_RESIDUAL)
                        out[row] = __float2half(__half2float(ex.residual[row]) + round_f16(v));
                    else
                        out[(size_t)a * M + row] = __float2half(v);
                }
            }
        }
        // `red` is rewritten only after the next tile's K loop and `part` alternates, so no
        // second barrier is needed here: a CTA can be at most one tile ahead of the leader's
        // reads, because the next tile's cluster barrier needs the leader too.
    };

    WeightRegs other;
    const int total = my_tiles * nsw;
    for (int e = 0; e < total; e += 2) {
        do_elem(cur, other);
        if (e + 1 < total) do_elem(other, cur);
    }
    if (S > 1) cluster_sync_all();   // no CTA may exit while a peer can still read its shared memory

    if (EPI == EPI_ALLREDUCE) {
        __shared__ uint32_t s_last, s_seq;
        unsigned char* mine = ex.comm[ex.rank];
        uint32_t* errw = reinterpret_cast<uint32_t*>(mine + 4);
        __threadfence_system();          // this CTA's peer stores before its "finished" count
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t* done = reinterpret_cast<uint32_t*>(mine + NVFP4_PUSH_DONE_OFF);
            const uint32_t prev = atomicAdd(done, 1u);
            s_last = (prev == gridDim.x - 1) ? 1u : 0u;
            if (s_last) {
                *done = 0u;
                uint32_t* seqp = reinterpret_cast<uint32_t*>(mine + NVFP4_PUSH_SEQ_OFF);
                s_seq = *seqp + 1u;
                *seqp = s_seq;
                __threadfence_system();  // every CTA's stores (seen through the counter) first
            }
        }
        __syncthreads();
        if (s_last) {
            const uint32_t seq = s_seq;
            const int tid = threadIdx.x;
            if (tid < ex.world && tid != ex.rank) {
                uint32_t* pf = reinterpret_cast<uint32_t*>(ex.comm[tid] + NVFP4_PUSH_FLAGS_OFF) +
                               ex.parity * 8 + ex.rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(pf), "r"(seq) : "memory");
                const uint32_t* mf = reinterpret_cast<const uint32_t*>(mine + NVFP4_PUSH_FLAGS_OFF) +
                                     ex.parity * 8 + tid;
                uint32_t spins = 0, v;
                do {
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(mf) : "memory");
                    if ((int32_t)(v - seq) >= 0) break;
                } while (++spins <= NVFP4_PUSH_SPIN_LIMIT);
                if ((int32_t)(v - seq) < 0) atomicExch(errw, 101u + (uint32_t)tid);
            }
            __syncthreads();
            // out[m] += f16(sum of the ranks' partial vectors), all now in THIS rank's buffer
            for (int i = tid * 8; i < M; i += WARPS * 32 * 8) {
                float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
                for (int r = 0; r < ex.world; r++) {
                    uint4 v;
                    const void* src = mine + push_data_off(ex.comm_n, ex.parity, r) +
                                      (size_t)i * sizeof(__half);
                    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                                 : "l"(src)
                                 : "memory");
                    const __half2* hp = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 f = __half22float2(hp[e]);
                        acc[2 * e] += f.x;
                        acc[2 * e + 1] += f.y;
                    }
                }
                uint4 hv = *reinterpret_cast<const uint4*>(out + i);
                __half2* hp = reinterpret_cast<__half2*>(&hv);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(hp[e]);
                    hp[e] = __floats2half2_rn(f.x + round_f16(acc[2 * e]),
                                              f.y + round_f16(acc[2 * e + 1]));
                }
                *reinterpret_cast<uint4*>(out + i) = hv;
            }
        }
    }
}

// Generic path for shapes or pointers the tensor-core kernel does not take (K % 128 != 0, or
// weaker alignment): one warp per row, 16-byte loads, fp32 FMA.  K % 32 == 0, packed and
// activations 16-byte aligned, scales 2-byte aligned.
// ILV (two activations): act0 holds K pairs (a0[k], a1[k]) instead of two separate vectors.
template <int NACT, bool ILV = false>
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
                uint32_t xw[4];
                if (ILV) {
                    const uint4* ip = reinterpret_cast<const uint4*>(act0 + (size_t)c * 64) + 2 * j;
                    const uint4 lo = __ldg(ip), hi = __ldg(ip + 1);
                    const uint32_t sel = a ? 0x7632u : 0x5410u;
                    xw[0] = __byte_perm(lo.x, lo.y, sel);
                    xw[1] = __byte_perm(lo.z, lo.w, sel);
                    xw[2] = __byte_perm(hi.x, hi.y, sel);
                    xw[3] = __byte_perm(hi.z, hi.w, sel);
                } else {
                    const uint4 xv = __ldg(xp + j);
                    xw[0] = xv.x; xw[1] = xv.y; xw[2] = xv.z; xw[3] = xv.w;
                }
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
    int max_split = 0;     // largest cluster K split the planner may pick (0 or 1 = none; 2; 4)
    int force_split = 0;   // 0 = planner decides; 1, 2 or 4 = use exactly this K split
};
static GemvConfig g_cfg;
constexpr int MAX_DEVICES = NVFP4_MAX_DEVICES;
static int current_device() { return current_device_index(); }

// SM count of the current device (a process may drive several GPUs: cached per device)
static int num_sms() {
    static int cache[MAX_DEVICES] = {0};
    const int dev = current_device();
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

// A caller that sets one of the register-streaming kernel's tuning values wants that kernel.
static bool old_kernel_tuned() {
    return g_cfg.warps || g_cfg.ctas_per_sm || g_cfg.max_split || g_cfg.force_split;
}

// Work partition of one GEMV: CTAs of `warps` warps, clusters of `split` CTAs that share a row
// tile's K range, `grid` CTAs in total.  Chosen so that every cluster gets the same number of
// tiles and as many of the machine's warp slots as possible are busy over whole rounds: a grid
// that simply filled every slot leaves most CTAs idle in its last round (1088 tiles on 888 slots:
// two rounds, the second 22 % full), and with few row tiles (M = 5120: 320) only the K split
// provides enough CTAs.
struct GemvPlan { int warps, split, grid; };

// force_warps (0, 4 or 8) and max_split (0 = the configured cap) override the process-wide tuning
// values for one call.
static GemvPlan plan_gemv(int M, int K, int force_warps = 0, int max_split = 0) {
    const int ntiles = (M + 15) / 16, nsteps = (K + 255) / 256;
    GemvPlan best = {4, 1, ntiles};
    double best_score = -1.0;
    const int want_warps = force_warps ? force_warps : g_cfg.warps;
    const int split_cap = max_split ? max_split : (g_cfg.max_split ? g_cfg.max_split : 1);
    for (int w = 4; w <= 8; w += 4) {
        if (want_warps && want_warps != w && (want_warps == 4 || want_warps == 8)) continue;
        const int slots = num_sms() * (24 / w);
        for (int sp = 1; sp <= 4; sp *= 2) {
            if (sp > split_cap && !g_cfg.force_split) continue;
            if (g_cfg.force_split && sp != g_cfg.force_split) continue;
            if (sp * w > nsteps && sp > 1 && !g_cfg.force_split) continue;  // nothing left to split
            const long long units = (long long)ntiles * sp;
            const int r = (int)((units + slots - 1) / slots);      // tiles per cluster
            const int clusters = (ntiles + r - 1) / r;
            const int grid = clusters * sp;
            const int nsw = (nsteps + sp * w - 1) / (sp * w);
            const double fill = (double)ntiles / ((double)r * clusters);
            double occ = (double)grid * w / (num_sms() * 24.0);
            if (occ > 1.0) occ = 1.0;
            const double kfill = (double)nsteps / ((double)nsw * sp * w);
            const double cost = (sp == 1) ? 1.0 : (sp == 2 ? 0.97 : 0.94);  // cluster barrier per tile
            const double score = fill * occ * kfill * cost;
            if (score > best_score + 1e-9) {
                best_score = score;
                best = {w, sp, grid};
            }
        }
    }
    // Measured exception to the equal-shares rule: when the tiles left over after whole rounds
    // are few (at most a third of the slots), filling every slot and letting a few CTAs run one
    // extra tile on an otherwise idle machine is faster than shrinking the grid for all rounds
    // (896 tiles on 444 slots: 14.0 us against 14.9 us).
    if (best.split == 1 && !g_cfg.force_split) {
        const int slots = num_sms() * (24 / best.warps);
        if (ntiles > slots && (ntiles % slots) * 3 <= slots) best.grid = slots;
    }
    return best;
}

template <int WARPS, int NACT, int PRO, int EPI>
static cudaError_t launch_mma(const void* packed, const void* scales, const void* a0, const void* a1,
                              void* out, int M, int K, cudaStream_t st, const GemvExtra& ex,
                              const GemvPlan& plan) {
    const int smem = (PRO == PRO_RMSNORM || PRO == PRO_AR_RMSNORM) ? K * 2
                     : (PRO == PRO_INTERLEAVED)                     ? K * 4 : 0;
    // the opt-in to more than 48 KB of dynamic shared memory applies to the current device only
    static int max_smem_set[MAX_DEVICES] = {0};
    const int dev = current_device();
    if (smem > 48 * 1024 && smem > max_smem_set[dev]) {
        if (cudaFuncSetAttribute(gemv_mma_kernel<WARPS, NACT, PRO, EPI>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return cudaErrorInvalidValue;
        max_smem_set[dev] = smem;
    }
    const int ntiles = (M + 15) / 16;
    int grid = plan.grid;
    if (g_cfg.ctas_per_sm > 64) {          // tuning: an exact grid size
        grid = g_cfg.ctas_per_sm;
        if (grid > ntiles * plan.split) grid = ntiles * plan.split;
        grid -= grid % plan.split;
        if (grid < plan.split) grid = plan.split;
    } else if (g_cfg.ctas_per_sm > 0) {
        grid = num_sms() * g_cfg.ctas_per_sm;
        if (grid > ntiles * plan.split) grid = ntiles * plan.split;
        grid -= grid % plan.split;
        if (grid < plan.split) grid = plan.split;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (!g_cfg.no_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    if (plan.split > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)plan.split;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, gemv_mma_kernel<WARPS, NACT, PRO, EPI>, (const uint8_t*)packed,
                              (const uint8_t*)scales, (const __half*)a0, (const __half*)a1,
                              (__half*)out, M, K, ex);
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
    StreamPlan sp;
    if (fast && nact == 1 && !old_kernel_tuned() && aligned(scales, 16) && nvfp4_gemv_tc_wanted_plain(M, K)) {
        // large matrices: the FP4 tensor-core kernel
        const int rc = launch_nvfp4_gemv_tc((const uint8_t*)packed, (const uint8_t*)scales, a0, out, M, K,
                                            stream);
        if (rc == 0) return NVFP4_OK;
        if (rc != NVFP4_ERR_SHAPE && rc != -3) {
            fprintf(stderr, "%s (tensor-core kernel): error %d\n", who, rc);
            return NVFP4_ERR_LAUNCH;
        }
    }
    if (fast && nact == 1 && !old_kernel_tuned() && aligned(scales, 16) &&
        plan_stream(M, K, GS_PRO_NONE, GS_EPI_STORE, &sp)) {
        e = launch_stream(packed, scales, a0, out, M, K, GS_PRO_NONE, nullptr, 0.0f, GS_EPI_STORE,
                          nullptr, sp, st, !g_cfg.no_pdl);
    } else if (fast) {
        GemvPlan plan = plan_gemv(M, K);
        if (g_cfg.warps == 2) plan = {2, 1, (M + 15) / 16 < num_sms() * 12 ? (M + 15) / 16 : num_sms() * 12};
        const int warps = plan.warps;
        GemvExtra none = {};
        if (nact == 1) {
            e = (warps == 8) ? launch_mma<8, 1, 0, 0>(packed, scales, a0, a1, out, M, K, st, none, plan)
              : (warps == 2) ? launch_mma<2, 1, 0, 0>(packed, scales, a0, a1, out, M, K, st, none, plan)
                             : launch_mma<4, 1, 0, 0>(packed, scales, a0, a1, out, M, K, st, none, plan);
        } else {
            if (plan.warps == 2) plan.warps = 4;
            e = (plan.warps == 8)
                    ? launch_mma<8, 2, 0, 0>(packed, scales, a0, a1, out, M, K, st, none, plan)
                    : launch_mma<4, 2, 0, 0>(packed, scales, a0, a1, out, M, K, st, none, plan);
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

// Two activations stored as K (a0[k], a1[k]) pairs; out[m] = W a0, out[M + m] = W a1.
int gemv2i_dispatch(const void* packed, const void* scales, const void* act_i, void* out, int M,
                    int K, void* stream) {
    if (K <= 0 || K % (NVFP4_BLOCK * 2) != 0) return NVFP4_ERR_SHAPE;
    if (M <= 0 || !packed || !scales || !act_i || !out) return NVFP4_ERR_SHAPE;
    if (!aligned(packed, 16) || !aligned(act_i, 16) || !aligned(scales, 2) || !aligned(out, 2))
        return NVFP4_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const bool fast = !g_cfg.force_generic && (K % 128 == 0) && aligned(packed, 32) &&
                      aligned(scales, 8) && K * 4 <= 200 * 1024;
    if (fast) {
        GemvPlan plan = plan_gemv(M, K);
        GemvExtra none = {};
        e = (plan.warps == 8)
                ? launch_mma<8, 2, PRO_INTERLEAVED, 0>(packed, scales, act_i, act_i, out, M, K, st, none, plan)
                : launch_mma<4, 2, PRO_INTERLEAVED, 0>(packed, scales, act_i, act_i, out, M, K, st, none, plan);
    } else {
        gemv_generic_kernel<2, true><<<(unsigned)((M + 7) / 8), 256, 0, st>>>(
            (const uint8_t*)packed, (const uint8_t*)scales, (const __half*)act_i,
            (const __half*)act_i, (__half*)out, M, K);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        fprintf(stderr, "launch_nvfp4_gemv2i launch: %s\n", cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return NVFP4_OK;
}

// Fused GEMV of the decode engine.  Only the tensor-core kernel implements the fusions, so the
// shape and alignment rules of that kernel are requirements here.
int gemv_ex_dispatch(const void* packed, const void* scales, const void* act, void* out, int M,
                     int K, int prologue, const void* norm_w1, float eps, int epilogue,
                     const void* residual, void* stream) {
    if (K <= 0 || K % 128 != 0 || M <= 0) return NVFP4_ERR_SHAPE;
    if (!packed || !scales || !act || !out) return NVFP4_ERR_SHAPE;
    if (!aligned(packed, 32) || !aligned(scales, 8) || !aligned(act, 16) || !aligned(out, 2))
        return NVFP4_ERR_SHAPE;
    if (prologue != PRO_NONE && prologue != PRO_RMSNORM) return NVFP4_ERR_SHAPE;
    if (prologue == PRO_RMSNORM && (!norm_w1 || !aligned(norm_w1, 16) || K * 2 > 200 * 1024))
        return NVFP4_ERR_SHAPE;
    if (epilogue < EPI_STORE || epilogue > EPI_SILU_MUL) return NVFP4_ERR_SHAPE;
    if (epilogue == EPI_RESIDUAL && !residual) return NVFP4_ERR_SHAPE;
    if (epilogue == EPI_SILU_MUL && M % 16 != 0) return NVFP4_ERR_SHAPE;
    // large matrices: the FP4 tensor-core kernel (TMA ring, no weight byte through a register)
    if (!old_kernel_tuned() && nvfp4_gemv_tc_wanted(M, K) && aligned(scales, 16)) {
        const int rc = launch_nvfp4_gemv_tc_fused((const uint8_t*)packed, (const uint8_t*)scales, act, out,
                                                  M, K, prologue, norm_w1, eps, epilogue, residual, stream);
        if (rc == 0) return NVFP4_OK;
        if (rc != NVFP4_ERR_SHAPE && rc != -3) {
            fprintf(stderr, "launch_nvfp4_gemv_fused (tensor-core kernel): error %d\n", rc);
            return NVFP4_ERR_LAUNCH;
        }
    }
    GemvExtra ex = {};
    ex.norm_w1 = (const float*)norm_w1;
    ex.eps = eps;
    ex.residual = (const __half*)residual;
    cudaStream_t st = (cudaStream_t)stream;
    StreamPlan sp;
    if (!old_kernel_tuned() && aligned(scales, 16) && plan_stream(M, K, prologue, epilogue, &sp)) {
        const cudaError_t es = launch_stream(packed, scales, act, out, M, K, prologue, norm_w1, eps,
                                             epilogue, residual, sp, st, !g_cfg.no_pdl);
        if (es != cudaSuccess) {
            fprintf(stderr, "launch_nvfp4_gemv_fused (ring): %s\n", cudaGetErrorString(es));
            return NVFP4_ERR_LAUNCH;
        }
        return NVFP4_OK;
    }
    GemvPlan plan = plan_gemv(M, K);
    if (prologue == PRO_RMSNORM) {
        // the prologue keeps PRO_NV vectors of 8 activations per thread
        if (K > PRO_NV * 8 * 256) return NVFP4_ERR_SHAPE;
        if (K > PRO_NV * 8 * 128 && plan.warps != 8) plan = plan_gemv(M, K, 8);
    }
    const int warps = plan.warps;
    cudaError_t e;
#define NVFP4_EX_CASE(P, E)                                                                     \
    e = (warps == 8)                                                                            \
            ? launch_mma<8, 1, P, E>(packed, scales, act, nullptr, out, M, K, st, ex, plan)     \
            : launch_mma<4, 1, P, E>(packed, scales, act, nullptr, out, M, K, st, ex, plan)
    if (prologue == PRO_NONE) {
        if (epilogue == EPI_STORE) { NVFP4_EX_CASE(0, 0); }
        else if (epilogue == EPI_RESIDUAL) { NVFP4_EX_CASE(0, 1); }
        else { NVFP4_EX_CASE(0, 2); }
    } else {
        if (epilogue == EPI_STORE) { NVFP4_EX_CASE(1, 0); }
        else if (epilogue == EPI_RESIDUAL) { NVFP4_EX_CASE(1, 1); }
        else { NVFP4_EX_CASE(1, 2); }
    }
#undef NVFP4_EX_CASE
    if (e != cudaSuccess) {
        fprintf(stderr, "launch_nvfp4_gemv_fused: %s\n", cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return NVFP4_OK;
}

// GEMV whose prologue first completes the all-reduce of the PREVIOUS K-split layer into the
// residual stream h, then RMS-normalises h (see PRO_AR_RMSNORM in the kernel).
int gemv_ar_in_dispatch(const void* packed, const void* scales, void* h, void* out, int M, int K,
                        const void* norm_w1, float eps, int epilogue, const void* const* bufs,
                        int rank, int world, int n, int parity, const void* epoch, int site,
                        int n_sites, void* stream) {
    if (K <= 0 || K % 128 != 0 || M <= 0 || K > n) return NVFP4_ERR_SHAPE;
    if (!packed || !scales || !h || !out || !norm_w1 || !bufs || !epoch) return NVFP4_ERR_SHAPE;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || n % 8 != 0 || site < 0 ||
        site >= n_sites)
        return NVFP4_ERR_SHAPE;
    if (!aligned(packed, 32) || !aligned(scales, 8) || !aligned(h, 16) || !aligned(out, 2) ||
        !aligned(norm_w1, 16) || K * 2 > 200 * 1024)
        return NVFP4_ERR_SHAPE;
    if (epilogue != EPI_STORE && epilogue != EPI_SILU_MUL) return NVFP4_ERR_SHAPE;
    if (epilogue == EPI_SILU_MUL && M % 16 != 0) return NVFP4_ERR_SHAPE;
    if (K > PRO_NV * 8 * 256) return NVFP4_ERR_SHAPE;
    GemvExtra ex = {};
    ex.norm_w1 = (const float*)norm_w1;
    ex.eps = eps;
    for (int r = 0; r < world; r++) {
        if (!bufs[r]) return NVFP4_ERR_SHAPE;
        ex.comm[r] = (unsigned char*)bufs[r];
    }
    ex.rank = rank;
    ex.world = world;
    ex.parity = parity & 1;
    ex.comm_n = n;
    ex.epoch = (const unsigned int*)epoch;
    ex.site = site;
    ex.n_sites = n_sites;
    // every CTA waits for CTA 0 inside the kernel, so all of them must be resident at once: the
    // planner's grids never exceed the resident slots, and the K split (clusters) is not used
    GemvPlan plan = plan_gemv(M, K, (K > PRO_NV * 8 * 128) ? 8 : 0, 1);
    plan.split = 1;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (epilogue == EPI_STORE)
        e = (plan.warps == 8)
                ? launch_mma<8, 1, PRO_AR_RMSNORM, EPI_STORE>(packed, scales, h, nullptr, out, M, K, st, ex, plan)
                : launch_mma<4, 1, PRO_AR_RMSNORM, EPI_STORE>(packed, scales, h, nullptr, out, M, K, st, ex, plan);
    else
        e = (plan.warps == 8)
                ? launch_mma<8, 1, PRO_AR_RMSNORM, EPI_SILU_MUL>(packed, scales, h, nullptr, out, M, K, st, ex, plan)
                : launch_mma<4, 1, PRO_AR_RMSNORM, EPI_SILU_MUL>(packed, scales, h, nullptr, out, M, K, st, ex, plan);
    if (e != cudaSuccess) {
        fprintf(stderr, "launch_nvfp4_gemv_fused_ar: %s\n", cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return NVFP4_OK;
}

// Tensor-parallel K-split layer: GEMV + all-reduce + residual add in one kernel.
int gemv_allreduce_dispatch(const void* packed, const void* scales, const void* act, void* h, int M,
                            int K, const void* const* bufs, int rank, int world, int n, int parity,
                            void* stream) {
    if (K <= 0 || K % 128 != 0 || M <= 0 || M % 16 != 0) return NVFP4_ERR_SHAPE;
    if (!packed || !scales || !act || !h || !bufs) return NVFP4_ERR_SHAPE;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || n < M || n % 8 != 0)
        return NVFP4_ERR_SHAPE;
    if (!aligned(packed, 32) || !aligned(scales, 8) || !aligned(act, 16) || !aligned(h, 16))
        return NVFP4_ERR_SHAPE;
    GemvExtra ex = {};
    for (int r = 0; r < world; r++) {
        if (!bufs[r]) return NVFP4_ERR_SHAPE;
        ex.comm[r] = (unsigned char*)bufs[r];
    }
    ex.rank = rank;
    ex.world = world;
    ex.parity = parity & 1;
    ex.comm_n = n;
    GemvPlan plan = plan_gemv(M, K, 0, 1);       // the finished-CTA count assumes one CTA per tile
    plan.split = 1;
    cudaStream_t st = (cudaStream_t)stream;
    const cudaError_t e =
        (plan.warps == 8)
            ? launch_mma<8, 1, 0, EPI_ALLREDUCE>(packed, scales, act, nullptr, h, M, K, st, ex, plan)
            : launch_mma<4, 1, 0, EPI_ALLREDUCE>(packed, scales, act, nullptr, h, M, K, st, ex, plan);
    if (e != cudaSuccess) {
        fprintf(stderr, "launch_nvfp4_gemv_allreduce: %s\n", cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return NVFP4_OK;
}

}  // namespace nvfp4

extern "C" {

// h[M] (fp16, in place) += f16( sum over the ranks of W_r[M, K] . act_r[K] ): a tensor-parallel
// K-split layer, its all-reduce and the residual add as ONE kernel over NVLink peer memory.
// bufs: HOST array of `world` device pointers, every rank's communication buffer as mapped here
// (see nvfp4_comm_buffer_bytes); n: the buffers' vector capacity (n >= M); parity alternates
// 0, 1, 0, ... over the calls; every rank makes the same sequence of calls.  No counterpart in
// the reference.  0; -2 bad arguments; -1 launch error.
int launch_nvfp4_gemv_allreduce(const void* weight_packed, const void* weight_scales,
                                const void* activation, void* h, int M, int K,
                                const void* const* bufs, int rank, int world, int n, int parity,
                                void* stream) {
    return nvfp4::gemv_allreduce_dispatch(weight_packed, weight_scales, activation, h, M, K, bufs,
                                          rank, world, n, parity, stream);
}

// Tensor-parallel consumer of a K-split layer (no counterpart in the reference): the all-reduce
// of that layer's partial vectors and the residual add run INSIDE this GEMV's prologue instead of
// in a kernel of their own.  h fp16 [K] (in/out): the residual stream, to which the sum over the
// ranks of the partial vectors in data slot `parity` of the communication buffers is added (by
// CTA 0, over NVLink peer loads, after a bounded flag exchange); every CTA then RMS-normalises the
// new h with norm_w1 and multiplies.  epilogue 0 or 2 as in launch_nvfp4_gemv_fused.  epoch: a
// device u32 counting decode steps (advanced by launch_argmax_exchange or by the caller), site /
// n_sites: this call's place among the all-reduces of one step, the same on every rank.
// 0; -2 bad arguments; -1 launch error.  A wait that ran out shows in nvfp4_comm_status (201 + r:
// peer r missing; 299: CTA 0 never published) and leaves h without the sum.
int launch_nvfp4_gemv_fused_ar(const void* weight_packed, const void* weight_scales, void* h,
                               void* output, int M, int K, const void* norm_w1, float eps,
                               int epilogue, const void* const* bufs, int rank, int world, int n,
                               int parity, const void* epoch, int site, int n_sites, void* stream) {
    return nvfp4::gemv_ar_in_dispatch(weight_packed, weight_scales, h, output, M, K, norm_w1, eps,
                                      epilogue, bufs, rank, world, n, parity, epoch, site, n_sites,
                                      stream);
}

// GEMV with optional fused RMSNorm of the activation (prologue = 1) and fused residual add
// (epilogue = 1) or silu(gate)*up over interleaved gate/up rows (epilogue = 2).  No counterpart in
// the reference, which launches those operators as separate kernels.
int launch_nvfp4_gemv_fused(const void* weight_packed, const void* weight_scales,
                            const void* activation, void* output, int M, int K, int prologue,
                            const void* norm_w1, float eps, int epilogue, const void* residual,
                            void* stream) {
    return nvfp4::gemv_ex_dispatch(weight_packed, weight_scales, activation, output, M, K,
                                   prologue, norm_w1, eps, epilogue, residual, stream);
}

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

// reference: kernels/nvfp4_gemv.cu:997-1011 (launch_nvfp4_gemv2i): two activations interleaved
// as K (a0[k], a1[k]) fp16 pairs; output [2, M].
int launch_nvfp4_gemv2i(const void* weight_packed, const void* weight_scales, const void* act_i,
                        void* output, int M, int K, void* stream) {
    return nvfp4::gemv2i_dispatch(weight_packed, weight_scales, act_i, output, M, K, stream);
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
        const int ms = (flags >> 4) & 7;   // bits 4..6: largest cluster K split (0 = planner decides)
        if (!(ms == 0 || ms == 1 || ms == 2 || ms == 4)) return NVFP4_ERR_SHAPE;
        nvfp4::g_cfg.max_split = ms;
        const int fs = (flags >> 8) & 7;   // bits 8..10: force this cluster K split
        if (!(fs == 0 || fs == 1 || fs == 2 || fs == 4)) return NVFP4_ERR_SHAPE;
        nvfp4::g_cfg.force_split = fs;
    }
    return NVFP4_OK;
}

}  // extern "C"

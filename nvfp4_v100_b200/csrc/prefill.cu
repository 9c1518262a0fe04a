// Chunked prefill around the tensor-core GEMM: everything a prompt chunk needs between the GEMMs,
// with the arithmetic (formulas and fp16 rounding points) of the decode-step kernels, so that a
// prompt fed through here leaves the KV cache, the conv window and the recurrent state as feeding
// it token by token through the decode step would, up to the GEMM-vs-GEMV summation order.
//
// The reference prefills through the third-party model code (pipeline/_qwen38_infer.py:796-809:
// 512-token chunks, every Linear running launch_nvfp4_gemmtc_v5, attention and the gated delta
// rule in PyTorch).  Here the chunk's activations are token-major [tokens][features] between the
// operators and token-minor [features][tokens] at the GEMM (its activation layout), with a
// transposing copy at each boundary:
//   transpose_f16 / add_transposed   layout changes (the second fused with the residual add)
//   embed_rows                       token ids -> embedding rows
//   silu_mul_rows                    gate/up rows (interleaved by 8) -> activation rows
//   dn_conv_tokens, dn_prep, dn_scan, dn_post   one Gated-DeltaNet layer over a chunk:
//       causal conv + silu over the chunk with the carried window; q/k L2 norm, beta, decay;
//       the recurrence S_t = S_{t-1} e^{g_t} + k_t (v_t - S_{t-1} e^{g_t} k_t) beta_t, o_t = S_t q_t
//       run sequentially over the chunk with every state row in registers (rows are independent:
//       8 lanes own a row, 16 dims each; 6144 rows of the full model are 768 warps); gated norm.
// Attention uses attn_prep_tokens_kernel (decode_ops.cu) and attn_prefill_group_kernel
// (fused_ops.cu).
#include <cstdio>

#include "common.cuh"

namespace nvfp4 {

__device__ __forceinline__ float silu_pf(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_pf(float x) { return (x > 20.0f) ? x : log1pf(expf(x)); }

// dst[c][r] = src[r][c] for r < R, c < C; dst rows are ld_dst long and columns R .. ld_dst-1 are
// zero-filled (the GEMM reads whole rows).  src rows are ld_src long.
__global__ void __launch_bounds__(256)
transpose_f16_kernel(const __half* __restrict__ src, long long ld_src, __half* __restrict__ dst,
                     long long ld_dst, int R, int C) {
    pdl_prologue();
    PDL_FRESH(src); PDL_FRESH(dst);
    __shared__ __half tile[64][66];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    // read 64 rows x 64 columns: a thread reads two adjacent columns (one 4-byte load)
    for (int i = ty; i < 64; i += 8) {
        const int r = r0 + i, c = c0 + tx * 2;
        __half2 v = __floats2half2_rn(0.0f, 0.0f);
        if (r < R) {
            if (c + 1 < C && ((ld_src | c) & 1) == 0) {
                v = *reinterpret_cast<const __half2*>(src + (size_t)r * ld_src + c);
            } else {
                const __half lo = (c < C) ? src[(size_t)r * ld_src + c] : __float2half(0.0f);
                const __half hi = (c + 1 < C) ? src[(size_t)r * ld_src + c + 1] : __float2half(0.0f);
                v = __halves2half2(lo, hi);
            }
        }
        tile[i][tx * 2] = __low2half(v);
        tile[i][tx * 2 + 1] = __high2half(v);
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 8) {
        const int c = c0 + i, r = r0 + tx * 2;
        if (c >= C) continue;
        __half* d = dst + (size_t)c * ld_dst + r;
        if (r + 1 < ld_dst && ((ld_dst | r) & 1) == 0) {
            *reinterpret_cast<__half2*>(d) = __halves2half2(tile[tx * 2][i], tile[tx * 2 + 1][i]);
        } else {
            if (r < ld_dst) d[0] = tile[tx * 2][i];
            if (r + 1 < ld_dst) d[1] = tile[tx * 2 + 1][i];
        }
    }
}

// h[t][c] = f16(f32(h[t][c]) + f32(dT[c][t])) for t < n, c < C: the residual add, reading the
// GEMM's token-minor output (rows ldT long).
__global__ void __launch_bounds__(256)
add_transposed_kernel(__half* __restrict__ h, const __half* __restrict__ dT, long long ldT, int n,
                      int C) {
    pdl_prologue();
    PDL_FRESH(h); PDL_FRESH(dT);
    __shared__ __half tile[64][66];
    const int t0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int i = ty; i < 64; i += 8) {          // rows of dT: feature c0 + i, tokens t0 ..
        const int c = c0 + i;
        const int t = t0 + tx * 2;
        __half lo = __float2half(0.0f), hi = lo;
        if (c < C) {
            if (t < n) lo = dT[(size_t)c * ldT + t];
            if (t + 1 < n) hi = dT[(size_t)c * ldT + t + 1];
        }
        tile[i][tx * 2] = lo;
        tile[i][tx * 2 + 1] = hi;
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 8) {          // rows of h: token t0 + i, features c0 ..
        const int t = t0 + i;
        if (t >= n) continue;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int c = c0 + tx * 2 + u;
            if (c < C) {
                __half* p = h + (size_t)t * C + c;
                *p = __float2half(__half2float(*p) + __half2float(tile[tx * 2 + u][i]));
            }
        }
    }
}

// out[t][:] = table[ids[t]][:]
__global__ void __launch_bounds__(256)
embed_rows_kernel(const __half* __restrict__ table, const long long* __restrict__ ids,
                  __half* __restrict__ out, int hidden, long long vocab) {
    pdl_prologue();
    PDL_FRESH(table); PDL_FRESH(ids); PDL_FRESH(out);
    long long id = ids[blockIdx.y];
    if (id < 0) id = 0;
    if (id >= vocab) id = vocab - 1;
    const int i = (blockIdx.x * 256 + threadIdx.x) * 8;
    const __half* src = table + (size_t)id * hidden;
    __half* dst = out + (size_t)blockIdx.y * hidden;
    if (i + 8 <= hidden && (hidden & 7) == 0) {
        *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
        for (int j = i; j < hidden && j < i + 8; j++) dst[j] = src[j];
    }
}

// Token-minor gate/up rows, interleaved in groups of 8 (rows 16j..16j+7 gate, 16j+8..16j+15 up),
// to activation rows: act[8j + r][t] = f16( f32(f16(silu(g))) * u ), the silu_mul_kernel chain.
__global__ void __launch_bounds__(256)
silu_mul_rows_kernel(const __half* __restrict__ gu, __half* __restrict__ act, int inter, int N) {
    pdl_prologue();
    PDL_FRESH(gu); PDL_FRESH(act);
    const int row = blockIdx.y;                       // activation row 0 .. inter-1
    const int t = (blockIdx.x * 256 + threadIdx.x) * 2;
    if (t >= N) return;
    const size_t grow = (size_t)(row >> 3) * 16 + (row & 7);
    const __half* g = gu + grow * N + t;
    const __half* u = gu + (grow + 8) * N + t;
    __half* o = act + (size_t)row * N + t;
    if (t + 1 < N && (N & 1) == 0) {
        const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(g));
        const float2 uf = __half22float2(*reinterpret_cast<const __half2*>(u));
        *reinterpret_cast<__half2*>(o) =
            __floats2half2_rn(round_f16(silu_pf(gf.x)) * uf.x, round_f16(silu_pf(gf.y)) * uf.y);
    } else {
        for (int k = t; k < N && k < t + 2; k++)
            act[(size_t)row * N + k] = __float2half(
                round_f16(silu_pf(__half2float(gu[grow * N + k]))) * __half2float(gu[(grow + 8) * N + k]));
    }
}

// ---------------------------------------------------------------------------------------------
// Gated DeltaNet over a chunk.  x: token-major in-projection output, row t =
// [ mixed (conv_dim = 2 key_dim + nv*128) | z (nv*128) | b (nv) | a (nv) ], ld halves per row.
// ---------------------------------------------------------------------------------------------
#define PF_DK 128

// conv[t][c] = f16(silu(w0 x[t-3] + w1 x[t-2] + w2 x[t-1] + w3 x[t])), inputs before the chunk
// taken from the carried window state[c][0..3] (state[c][3] is the newest).
__global__ void __launch_bounds__(256)
dn_conv_tokens_kernel(const __half* __restrict__ x, long long ld, const __half* __restrict__ conv_w,
                      const __half* __restrict__ conv_state, __half* __restrict__ conv_out,
                      int conv_dim) {
    pdl_prologue();
    PDL_FRESH(x); PDL_FRESH(conv_w); PDL_FRESH(conv_state); PDL_FRESH(conv_out);
    const int c = blockIdx.x * 256 + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= conv_dim) return;
    float win[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int tt = t - 3 + j;    // input index of tap j
        win[j] = (tt >= 0) ? __half2float(x[(size_t)tt * ld + c])
                           : __half2float(conv_state[(size_t)c * 4 + 4 + tt]);
    }
    const __half* w = conv_w + (size_t)c * 4;
    float acc = __half2float(w[0]) * win[0];
    acc = fmaf(__half2float(w[1]), win[1], acc);
    acc = fmaf(__half2float(w[2]), win[2], acc);
    acc = fmaf(__half2float(w[3]), win[3], acc);
    conv_out[(size_t)t * conv_dim + c] = __float2half(silu_pf(acc));
}

// carried window after the chunk: the last four inputs
__global__ void __launch_bounds__(256)
dn_conv_state_kernel(const __half* __restrict__ x, long long ld, __half* __restrict__ conv_state,
                     int conv_dim, int n) {
    pdl_prologue();
    PDL_FRESH(x); PDL_FRESH(conv_state);
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= conv_dim) return;
    __half old[4], nw[4];
#pragma unroll
    for (int j = 0; j < 4; j++) old[j] = conv_state[(size_t)c * 4 + j];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int tt = n - 4 + j;
        nw[j] = (tt >= 0) ? x[(size_t)tt * ld + c] : old[4 + tt];
    }
#pragma unroll
    for (int j = 0; j < 4; j++) conv_state[(size_t)c * 4 + j] = nw[j];
}

// per (token, key head): L2-normalised q (x 128^-1/2) and k as fp32; per (token, value head):
// beta = f16(sigmoid(b)), decay e^g with g = -exp(A_log) softplus(a + dt_bias).
// grid (nk + ceil(nv/32), n); 32 threads.
__global__ void __launch_bounds__(32)
dn_prep_kernel(const __half* __restrict__ conv_out, int conv_dim, const __half* __restrict__ x,
               long long ld, const __half* __restrict__ A_log, const __half* __restrict__ dt_bias,
               float* __restrict__ qn, float* __restrict__ kn, float2* __restrict__ be, int nk,
               int nv) {
    pdl_prologue();
    PDL_FRESH(conv_out); PDL_FRESH(x); PDL_FRESH(A_log); PDL_FRESH(dt_bias); PDL_FRESH(qn); PDL_FRESH(kn);
    PDL_FRESH(be);
    const int t = blockIdx.y, lane = threadIdx.x;
    const int key_dim = nk * PF_DK;
    if ((int)blockIdx.x < nk) {
        const int kh = blockIdx.x;
        const __half* row = conv_out + (size_t)t * conv_dim;
        float4 qv, kv;
        {
            const uint2 a = *reinterpret_cast<const uint2*>(row + kh * PF_DK + lane * 4);
            const uint2 b = *reinterpret_cast<const uint2*>(row + key_dim + kh * PF_DK + lane * 4);
            const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&a.x));
            const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
            const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&b.x));
            const float2 b1 = __half22float2(*reinterpret_cast<const __half2*>(&b.y));
            qv = make_float4(a0.x, a0.y, a1.x, a1.y);
            kv = make_float4(b0.x, b0.y, b1.x, b1.y);
        }
        const float qss = warp_sum(qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w);
        const float kss = warp_sum(kv.x * kv.x + kv.y * kv.y + kv.z * kv.z + kv.w * kv.w);
        const float inv_q = rsqrtf(qss + 1e-6f) * 0.08838834764831845f;
        const float inv_k = rsqrtf(kss + 1e-6f);
        qv.x *= inv_q; qv.y *= inv_q; qv.z *= inv_q; qv.w *= inv_q;
        kv.x *= inv_k; kv.y *= inv_k; kv.z *= inv_k; kv.w *= inv_k;
        const size_t o = ((size_t)t * nk + kh) * PF_DK + lane * 4;
        *reinterpret_cast<float4*>(qn + o) = qv;
        *reinterpret_cast<float4*>(kn + o) = kv;
    } else {
        const int h = ((int)blockIdx.x - nk) * 32 + lane;
        if (h >= nv) return;
        const __half* row = x + (size_t)t * ld + conv_dim + (size_t)nv * PF_DK;
        const float beta = round_f16(1.0f / (1.0f + expf(-__half2float(row[h]))));
        const float g = -expf(__half2float(A_log[h])) *
                        softplus_pf(__half2float(row[nv + h]) + __half2float(dt_bias[h]));
        be[(size_t)t * nv + h] = make_float2(beta, expf(g));
    }
}

// The recurrence over the chunk.  CTA = 4 warps = 16 state rows of one value head (384 CTAs for
// the full model: two or three per SM); a warp owns 4 rows, one per 8-lane group gi = lane >> 3;
// lane sub = lane & 7 owns dims 32 j + 4 sub .. + 3 (j = 0..3) of its row, so the 8 lanes of a
// group read one contiguous 128-byte piece of a vector at a time.  The operands of SCAN_TB tokens (the head's
// normalised k and q, this CTA's 32 values of v, beta and decay) are staged in shared memory by
// cp.async, double buffered, so the sequential chain never waits on global memory.
// o[t][h*128 + row] = f16(S_t[row] . q_t).
#define SCAN_WARPS 4
#define SCAN_RPG 1                          // state rows per 8-lane group
#define SCAN_ROWS (SCAN_WARPS * 4 * SCAN_RPG)
#define SCAN_TB 16

// packed fp32 pair arithmetic (two IEEE fp32 operations per instruction)
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(*reinterpret_cast<unsigned long long*>(&d))
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(*reinterpret_cast<unsigned long long*>(&d))
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return d;
}

struct ScanStage {
    float k[SCAN_TB][PF_DK];
    float q[SCAN_TB][PF_DK];
    __half v[SCAN_TB][SCAN_ROWS];
    float2 be[SCAN_TB];
};

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__global__ void __launch_bounds__(SCAN_WARPS * 32)
dn_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn,
               const float2* __restrict__ be, const __half* __restrict__ conv_out, int conv_dim,
               float* __restrict__ state, __half* __restrict__ o_out, int nk, int nv, int n) {
    pdl_prologue();
    PDL_FRESH(qn); PDL_FRESH(kn); PDL_FRESH(be); PDL_FRESH(conv_out); PDL_FRESH(state); PDL_FRESH(o_out);
    __shared__ __align__(16) ScanStage stage[2];
    const int per_head = PF_DK / SCAN_ROWS;                  // CTAs per value head
    const int h = blockIdx.x / per_head, part = blockIdx.x % per_head;
    const int kh = h / (nv / nk);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gi = lane >> 3, sub = lane & 7;
    const int lrow = (warp * 4 + gi) * SCAN_RPG;             // first of this lane's rows, in the CTA
    const int row0 = part * SCAN_ROWS + lrow;
    const int key_dim = nk * PF_DK;

    // stage the operands of tokens [t0, t0 + SCAN_TB) (clamped to the chunk) into buffer b
    auto issue = [&](int t0, int b) {
        ScanStage& s = stage[b];
        for (int i = tid; i < SCAN_TB * (PF_DK / 4); i += SCAN_WARPS * 32) {   // 16-byte pieces
            const int tt = i / (PF_DK / 4), c = i % (PF_DK / 4);
            const int t = min(t0 + tt, n - 1);
            const size_t o = ((size_t)t * nk + kh) * PF_DK + c * 4;
            cp_async_16(&s.k[tt][c * 4], kn + o);
            cp_async_16(&s.q[tt][c * 4], qn + o);
        }
        if (tid < SCAN_TB * (SCAN_ROWS / 8)) {
            const int tt = tid / (SCAN_ROWS / 8), c = tid % (SCAN_ROWS / 8);
            const int t = min(t0 + tt, n - 1);
            cp_async_16(&s.v[tt][c * 8], conv_out + (size_t)t * conv_dim + 2 * key_dim + h * PF_DK +
                                             part * SCAN_ROWS + c * 8);
        }
        if (tid >= 64 && tid < 64 + SCAN_TB) {
            const int tt = tid - 64;
            s.be[tt] = be[(size_t)min(t0 + tt, n - 1) * nv + h];
        }
        cp_async_commit();
    };

    __align__(8) float S[SCAN_RPG][16];
    float* sp = state + ((size_t)h * PF_DK + row0) * PF_DK + sub * 4;
#pragma unroll
    for (int r = 0; r < SCAN_RPG; r++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float4 v = *reinterpret_cast<const float4*>(sp + (size_t)r * PF_DK + j * 32);
            S[r][4 * j] = v.x; S[r][4 * j + 1] = v.y; S[r][4 * j + 2] = v.z; S[r][4 * j + 3] = v.w;
        }

    const int nblk = (n + SCAN_TB - 1) / SCAN_TB;
    if (nblk > 0) issue(0, 0);
    for (int blk = 0; blk < nblk; blk++) {
        const int cur = blk & 1;
        if (blk + 1 < nblk) {
            issue((blk + 1) * SCAN_TB, cur ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const ScanStage& s = stage[cur];
        const int tcount = min(SCAN_TB, n - blk * SCAN_TB);
        for (int tt = 0; tt < tcount; tt++) {
            // the row's 16 state values, k and q as 8 fp32 pairs: packed fp32x2 multiply-adds
            // halve the instruction count of the scan, which is issue-bound
            float2 kc[8], qc[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4 a = *reinterpret_cast<const float4*>(&s.k[tt][j * 32 + sub * 4]);
                const float4 c = *reinterpret_cast<const float4*>(&s.q[tt][j * 32 + sub * 4]);
                kc[2 * j] = make_float2(a.x, a.y); kc[2 * j + 1] = make_float2(a.z, a.w);
                qc[2 * j] = make_float2(c.x, c.y); qc[2 * j + 1] = make_float2(c.z, c.w);
            }
            const float2 bd = s.be[tt];
            const float beta = bd.x;
            const float2 eg2 = make_float2(bd.y, bd.y);
            float vr[SCAN_RPG], kvp[SCAN_RPG], od[SCAN_RPG];
#pragma unroll
            for (int r = 0; r < SCAN_RPG; r++) vr[r] = __half2float(s.v[tt][lrow + r]);
#pragma unroll
            for (int r = 0; r < SCAN_RPG; r++) {
                float2* S2 = reinterpret_cast<float2*>(S[r]);
                float2 a[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {            // four independent partial sums (pairs)
                    S2[2 * j] = fmul2(S2[2 * j], eg2);
                    S2[2 * j + 1] = fmul2(S2[2 * j + 1], eg2);
                    a[j] = fmul2(S2[2 * j], kc[2 * j]);
                    a[j] = ffma2(S2[2 * j + 1], kc[2 * j + 1], a[j]);
                }
                kvp[r] = ((a[0].x + a[0].y) + (a[1].x + a[1].y)) + ((a[2].x + a[2].y) + (a[3].x + a[3].y));
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1)
#pragma unroll
                for (int r = 0; r < SCAN_RPG; r++) kvp[r] += __shfl_xor_sync(0xffffffffu, kvp[r], o);
#pragma unroll
            for (int r = 0; r < SCAN_RPG; r++) {
                float2* S2 = reinterpret_cast<float2*>(S[r]);
                const float delta = (vr[r] - kvp[r]) * beta;
                const float2 d2 = make_float2(delta, delta);
                float2 a[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    S2[2 * j] = ffma2(kc[2 * j], d2, S2[2 * j]);
                    S2[2 * j + 1] = ffma2(kc[2 * j + 1], d2, S2[2 * j + 1]);
                    a[j] = fmul2(S2[2 * j], qc[2 * j]);
                    a[j] = ffma2(S2[2 * j + 1], qc[2 * j + 1], a[j]);
                }
                od[r] = ((a[0].x + a[0].y) + (a[1].x + a[1].y)) + ((a[2].x + a[2].y) + (a[3].x + a[3].y));
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1)
#pragma unroll
                for (int r = 0; r < SCAN_RPG; r++) od[r] += __shfl_xor_sync(0xffffffffu, od[r], o);
            if (sub == 0) {
#pragma unroll
                for (int r = 0; r < SCAN_RPG; r++)
                    o_out[((size_t)(blk * SCAN_TB + tt) * nv + h) * PF_DK + row0 + r] =
                        __float2half(od[r]);
            }
        }
        __syncthreads();     // everyone is done with this buffer before it is refilled
    }
#pragma unroll
    for (int r = 0; r < SCAN_RPG; r++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            *reinterpret_cast<float4*>(sp + (size_t)r * PF_DK + j * 32) =
                make_float4(S[r][4 * j], S[r][4 * j + 1], S[r][4 * j + 2], S[r][4 * j + 3]);
}

// gated norm per (token, value head): out = f16( f32(f16(o rsqrt(mean(o^2) + eps)) * norm_w) * silu(z) )
// grid (nv, n), 32 threads, lane owns 4 of the head's 128 outputs.
__global__ void __launch_bounds__(32)
dn_post_kernel(const __half* __restrict__ o_in, const __half* __restrict__ x, long long ld,
               int conv_dim, const __half* __restrict__ norm_w, __half* __restrict__ out, int nv,
               float rms_eps) {
    pdl_prologue();
    PDL_FRESH(o_in); PDL_FRESH(x); PDL_FRESH(norm_w); PDL_FRESH(out);
    const int h = blockIdx.x, t = blockIdx.y, lane = threadIdx.x;
    const uint2 ov = *reinterpret_cast<const uint2*>(o_in + ((size_t)t * nv + h) * PF_DK + lane * 4);
    const __half* oh = reinterpret_cast<const __half*>(&ov);
    float o[4], ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        o[j] = __half2float(oh[j]);
        ss = fmaf(o[j], o[j], ss);
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)PF_DK + rms_eps);
    const __half* z = x + (size_t)t * ld + conv_dim + (size_t)h * PF_DK + lane * 4;
    __half res[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const __half hw = __hmul(__float2half(o[j] * inv), norm_w[lane * 4 + j]);
        res[j] = __float2half(__half2float(hw) * silu_pf(__half2float(z[j])));
    }
    *reinterpret_cast<uint2*>(out + ((size_t)t * nv + h) * PF_DK + lane * 4) =
        *reinterpret_cast<const uint2*>(res);
}

}  // namespace nvfp4

extern "C" {

// dst[c][r] = src[r][c], r < R, c < C; dst rows ld_dst >= R long, the tail zero-filled.
int launch_transpose_f16(const void* src, long long ld_src, void* dst, long long ld_dst, int R,
                         int C, void* stream) {
    if (!src || !dst || R <= 0 || C <= 0 || ld_src < C || ld_dst < R) return -1;
    const dim3 grid((C + 63) / 64, (unsigned)((ld_dst + 63) / 64));
    return nvfp4::launch_pdl(nvfp4::transpose_f16_kernel, grid, dim3(256), 0, (cudaStream_t)stream,
                             (const __half*)src, ld_src, (__half*)dst, ld_dst, R, C) == cudaSuccess
               ? 0 : -1;
}

// h[t][c] += dT[c][t] (fp32 add, one fp16 rounding), t < n, c < C; h rows C long, dT rows ldT long.
int launch_add_transposed(void* h, const void* dT, long long ldT, int n, int C, void* stream) {
    if (!h || !dT || n <= 0 || C <= 0 || ldT < n) return -1;
    const dim3 grid((n + 63) / 64, (C + 63) / 64);
    return nvfp4::launch_pdl(nvfp4::add_transposed_kernel, grid, dim3(256), 0, (cudaStream_t)stream,
                             (__half*)h, (const __half*)dT, ldT, n, C) == cudaSuccess ? 0 : -1;
}

// out[t][0..hidden) = table[ids[t]], ids: device int64 [n].
int launch_embed_rows(const void* table, const void* ids, void* out, int n, int hidden,
                      long long vocab, void* stream) {
    if (!table || !ids || !out || n <= 0 || n > 65535 || hidden <= 0 || vocab <= 0) return -1;
    const dim3 grid((hidden + 2047) / 2048, n);
    return nvfp4::launch_pdl(nvfp4::embed_rows_kernel, grid, dim3(256), 0, (cudaStream_t)stream,
                             (const __half*)table, (const long long*)ids, (__half*)out, hidden,
                             vocab) == cudaSuccess ? 0 : -1;
}

// gu: token-minor [2 * inter][N] with gate/up rows interleaved in groups of 8; act: [inter][N].
int launch_silu_mul_rows(const void* gu, void* act, int inter, int N, void* stream) {
    if (!gu || !act || inter <= 0 || inter % 8 != 0 || inter > 65535 || N <= 0) return -1;
    const dim3 grid((N + 511) / 512, inter);
    return nvfp4::launch_pdl(nvfp4::silu_mul_rows_kernel, grid, dim3(256), 0, (cudaStream_t)stream,
                             (const __half*)gu, (__half*)act, inter, N) == cudaSuccess ? 0 : -1;
}

// Bytes of workspace launch_dn_prefill needs for n tokens.
long long nvfp4_dn_prefill_work_bytes(int n, int nk, int nv) {
    if (n <= 0 || nk <= 0 || nv <= 0) return -1;
    const long long conv_dim = (2LL * nk + nv) * PF_DK;
    long long b = (long long)n * conv_dim * 2;            // conv output, fp16
    b = (b + 255) & ~255LL;
    b += 2LL * n * nk * PF_DK * 4;                         // normalised q and k, fp32
    b += (long long)n * nv * 8;                            // (beta, decay)
    b = (b + 255) & ~255LL;
    b += (long long)n * nv * PF_DK * 2;                    // recurrence output, fp16
    return b + 256;
}

// One Gated-DeltaNet layer over a chunk of n tokens.  x: token-major in-projection output
// [n][ld], row = [mixed | z | b | a]; conv_w, conv_state fp16 [conv_dim][4]; A_log, dt_bias fp16
// [nv]; norm_w fp16 [128]; state fp32 [nv][128][128] (value-row major), updated; out token-major
// [n][nv * 128].  nv a multiple of nk.  Five launches on `stream`.  0; -1 bad arguments; -2 launch.
int launch_dn_prefill(const void* x, long long ld, const void* conv_w, void* conv_state,
                      const void* A_log, const void* dt_bias, const void* norm_w, void* state,
                      void* work, long long work_bytes, void* out, int n, int nk, int nv,
                      float rms_eps, void* stream) {
    if (!x || !conv_w || !conv_state || !A_log || !dt_bias || !norm_w || !state || !work || !out)
        return -1;
    if (n <= 0 || n > 65535 || nk <= 0 || nv <= 0 || nv % nk != 0) return -1;
    const int conv_dim = (2 * nk + nv) * PF_DK;
    if (ld < (long long)conv_dim + (long long)nv * PF_DK + 2LL * nv || (ld & 3)) return -1;
    if (work_bytes < nvfp4_dn_prefill_work_bytes(n, nk, nv) || ((uintptr_t)work & 255)) return -1;
    unsigned char* w = (unsigned char*)work;
    __half* conv_out = (__half*)w;
    long long off = ((long long)n * conv_dim * 2 + 255) & ~255LL;
    float* qn = (float*)(w + off);
    float* kn = qn + (size_t)n * nk * PF_DK;
    off += 2LL * n * nk * PF_DK * 4;
    float2* be = (float2*)(w + off);
    off = (off + (long long)n * nv * 8 + 255) & ~255LL;
    __half* o16 = (__half*)(w + off);
    cudaStream_t st = (cudaStream_t)stream;
    const __half* xh = (const __half*)x;
    bool ok = true;
    ok = ok && nvfp4::launch_pdl(nvfp4::dn_conv_tokens_kernel, dim3((conv_dim + 255) / 256, n),
                                 dim3(256), 0, st, xh, ld, (const __half*)conv_w,
                                 (const __half*)conv_state, conv_out, conv_dim) == cudaSuccess;
    ok = ok && nvfp4::launch_pdl(nvfp4::dn_conv_state_kernel, dim3((conv_dim + 255) / 256),
                                 dim3(256), 0, st, xh, ld, (__half*)conv_state, conv_dim,
                                 n) == cudaSuccess;
    ok = ok && nvfp4::launch_pdl(nvfp4::dn_prep_kernel, dim3(nk + (nv + 31) / 32, n), dim3(32), 0,
                                 st, (const __half*)conv_out, conv_dim, xh, ld,
                                 (const __half*)A_log, (const __half*)dt_bias, qn, kn, be, nk,
                                 nv) == cudaSuccess;
    ok = ok && nvfp4::launch_pdl(nvfp4::dn_scan_kernel, dim3(nv * (PF_DK / SCAN_ROWS)),
                                 dim3(SCAN_WARPS * 32), 0, st, (const float*)qn, (const float*)kn,
                                 (const float2*)be, (const __half*)conv_out, conv_dim,
                                 (float*)state, o16, nk, nv, n) == cudaSuccess;
    ok = ok && nvfp4::launch_pdl(nvfp4::dn_post_kernel, dim3(nv, n), dim3(32), 0, st,
                                 (const __half*)o16, xh, ld, conv_dim, (const __half*)norm_w,
                                 (__half*)out, nv, rms_eps) == cudaSuccess;
    return ok ? 0 : -2;
}

}  // extern "C"

// Decode-step elementwise / attention / DeltaNet kernels for sm_100a behind the reference's
// launcher signatures:
//   launch_rmsnorm      (reference: kernels/nvfp4_rmsnorm.cu:26-76)
//   launch_rope_qk      (reference: kernels/nvfp4_rope_silu.cu:29-53,70-81)
//   launch_silu_mul     (reference: kernels/nvfp4_rope_silu.cu:56-67,83-91)
//   launch_attn_decode  (reference: kernels/nvfp4_attn_decode.cu:29-132)
//   launch_dn_fused     (reference: kernels/nvfp4_dn_fused.cu:55-176)
// Each kernel keeps the reference's fp16 rounding points (where a value passes through an fp16
// tensor in the model it is rounded to fp16 here as well) and computes everything else in fp32.
// Reductions are warp-shuffle trees, so fp32 sums may differ from the reference's thread order in
// the last bit before the final fp16 rounding.
#include <cstdio>

#include "common.cuh"

namespace nvfp4 {

// ---------------------------------------------------------------------------------------------
// RMSNorm (zero-centred weight): out = f16( f32(x) * rsqrt(mean(x^2) + eps) * w1 ), w1 = 1 + w.
// One CTA per row; rows may be strided (row_stride elements between row starts).
// ---------------------------------------------------------------------------------------------
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_kernel(const __half* __restrict__ x, long long row_stride, const float* __restrict__ w1,
               __half* __restrict__ out, int n, float eps) {
    pdl_prologue();
    PDL_FRESH(x); PDL_FRESH(w1); PDL_FRESH(out);
    __shared__ float s_red[THREADS / 32];
    __shared__ float s_inv;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const __half* xr = x + (size_t)blockIdx.x * (size_t)row_stride;
    __half* orow = out + (size_t)blockIdx.x * (size_t)n;
    // 8 elements per thread per pass when both rows are 16-byte aligned
    const bool vec = ((n & 7) == 0) && ((((uintptr_t)xr) | ((uintptr_t)orow)) & 15) == 0 &&
                     ((((uintptr_t)w1) & 15) == 0);
    float ss = 0.0f;
    if (vec) {
        for (int i = t * 8; i < n; i += THREADS * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(h[j]);
                ss = fmaf(f.x, f.x, ss);
                ss = fmaf(f.y, f.y, ss);
            }
        }
    } else {
        for (int i = t; i < n; i += THREADS) {
            const float v = __half2float(xr[i]);
            ss = fmaf(v, v, ss);
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = (lane < THREADS / 32) ? s_red[lane] : 0.0f;
        v = warp_sum(v);
        if (lane == 0) s_inv = rsqrtf(v / (float)n + eps);
    }
    __syncthreads();
    const float inv = s_inv;
    if (vec) {
        for (int i = t * 8; i < n; i += THREADS * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
            const float4 wa = *reinterpret_cast<const float4*>(w1 + i);
            const float4 wb = *reinterpret_cast<const float4*>(w1 + i + 4);
            const __half2* h = reinterpret_cast<const __half2*>(&v);
            const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(h[j]);
                oh[j] = __halves2half2(__float2half(f.x * inv * w[2 * j]),
                                       __float2half(f.y * inv * w[2 * j + 1]));
            }
            *reinterpret_cast<uint4*>(orow + i) = o;
        }
    } else {
        for (int i = t; i < n; i += THREADS)
            orow[i] = __float2half(__half2float(xr[i]) * inv * w1[i]);
    }
}

// ---------------------------------------------------------------------------------------------
// RoPE on q [hq][256] and k [hkv][256] (full rotation, rotate_half = (-x2, x1)):
//   out = f16( f32(f16(v*c)) + f32(f16(rot(v)*s)) ).  One CTA per head, 128 threads, 2 dims each.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
rope_qk_kernel(const __half* __restrict__ q, const __half* __restrict__ k,
               const __half* __restrict__ cs, const __half* __restrict__ sn,
               __half* __restrict__ q_out, __half* __restrict__ k_out, int hq) {
    pdl_prologue();
    PDL_FRESH(q); PDL_FRESH(k); PDL_FRESH(cs); PDL_FRESH(sn); PDL_FRESH(q_out); PDL_FRESH(k_out);
    const int h = blockIdx.x, d = threadIdx.x;  // d in [0,128): handles d and d+128
    const bool is_q = h < hq;
    const size_t off = (size_t)(is_q ? h : h - hq) * 256;
    const __half* src = is_q ? q + off : k + off;
    __half* dst = is_q ? q_out + off : k_out + off;
    const float x1 = __half2float(src[d]), x2 = __half2float(src[d + 128]);
    const float c1 = __half2float(cs[d]), c2 = __half2float(cs[d + 128]);
    const float s1 = __half2float(sn[d]), s2 = __half2float(sn[d + 128]);
    const float lo = round_f16(x1 * c1) + round_f16(-x2 * s1);
    const float hi = round_f16(x2 * c2) + round_f16(x1 * s2);
    dst[d] = __float2half(lo);
    dst[d + 128] = __float2half(hi);
}

// ---------------------------------------------------------------------------------------------
// silu(g) * u with the model's rounding chain: s = f16(g / (1 + expf(-g))), out = f16(f32(s) * u).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half* __restrict__ g, const __half* __restrict__ u,
                __half* __restrict__ out, int n) {
    pdl_prologue();
    PDL_FRESH(g); PDL_FRESH(u); PDL_FRESH(out);
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const float gf = __half2float(g[i]), uf = __half2float(u[i]);
    out[i] = __float2half(round_f16(silu_f(gf)) * uf);
}

// ---------------------------------------------------------------------------------------------
// GQA attention decode (T = 1) over a static KV cache + sigmoid output gate.
//   q [HQ][256], keys/values [HKV][max_len][256] fp16, L = *cum_len (current token included),
//   gate [HQ][256]; out[h][d] = f16( f32(f16(o)) * f32(f16(sigmoid(gate))) ).
// One CTA per query head, 32 warps.  Keys are dealt to warps round-robin; a 512-byte key or value
// row is one coalesced warp read (16 bytes per lane), and each warp keeps 4 rows in flight.
// Pass 1: fp32 dot product + shuffle reduction, scores to shared memory.  Softmax in fp32 with
// expf (p_i = expf(s_i - max) * (1 / sum), as the reference computes it).  Pass 2: each lane owns
// 8 head dims and accumulates p_i * v_i over its warp's keys; the warps' partial sums are
// added in shared memory.  max_len is a run-time argument; the score buffer is dynamic shared
// memory (4 bytes per key).
// ---------------------------------------------------------------------------------------------
#define ATT_D 256
#define ATT_THREADS 1024
#define ATT_WARPS (ATT_THREADS / 32)

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 x = __half22float2(h[j]);
        f[2 * j] = x.x;
        f[2 * j + 1] = x.y;
    }
}

// One query head against the first L cache rows of its KV head; q, gate and out point at the
// head-major [heads][256] vectors of ONE token.
__device__ __forceinline__ void attn_one_query(const __half* __restrict__ q,
                                               const __half* __restrict__ keys,
                                               const __half* __restrict__ values, int L,
                                               const __half* __restrict__ gate,
                                               __half* __restrict__ out, int max_len, int gqa,
                                               float scale) {
    extern __shared__ float s_sc[];  // [max_len]
    __shared__ float s_red[ATT_WARPS];
    __shared__ float s_bcast;
    __shared__ float s_o[ATT_WARPS][ATT_D];
    const int h = blockIdx.x, kv = h / gqa;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;

    float qf[8];
    unpack8(*reinterpret_cast<const uint4*>(q + (size_t)h * ATT_D + lane * 8), qf);
    const __half* kbase = keys + (size_t)kv * (size_t)max_len * ATT_D + lane * 8;
    float m = -3.4e38f;
    for (int i0 = warp; i0 < L; i0 += ATT_WARPS * 4) {
        uint4 kr[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * ATT_WARPS;
            kr[u] = (i < L) ? *reinterpret_cast<const uint4*>(kbase + (size_t)i * ATT_D)
                            : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * ATT_WARPS;
            float kf[8];
            unpack8(kr[u], kf);
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) acc = fmaf(qf[j], kf[j], acc);
            acc = warp_sum(acc) * scale;
            if (i < L) {
                if (lane == 0) s_sc[i] = acc;
                m = fmaxf(m, acc);
            }
        }
    }
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    if (warp == 0) {
        float v = (lane < ATT_WARPS) ? s_red[lane] : -3.4e38f;
        v = warp_max(v);
        if (lane == 0) s_bcast = v;
    }
    __syncthreads();
    m = s_bcast;
    float l = 0.0f;
    for (int i = t; i < L; i += ATT_THREADS) {
        const float e = expf(s_sc[i] - m);
        s_sc[i] = e;
        l += e;
    }
    l = warp_sum(l);
    __syncthreads();  // s_red / s_bcast reuse
    if (lane == 0) s_red[warp] = l;
    __syncthreads();
    if (warp == 0) {
        float v = (lane < ATT_WARPS) ? s_red[lane] : 0.0f;
        v = warp_sum(v);
        if (lane == 0) s_bcast = 1.0f / v;
    }
    __syncthreads();
    const float inv_l = s_bcast;

    const __half* vbase = values + (size_t)kv * (size_t)max_len * ATT_D + lane * 8;
    float o[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    for (int i0 = warp; i0 < L; i0 += ATT_WARPS * 4) {
        uint4 vr[4];
        float p[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * ATT_WARPS;
            const bool ok = i < L;
            vr[u] = ok ? *reinterpret_cast<const uint4*>(vbase + (size_t)i * ATT_D)
                       : make_uint4(0u, 0u, 0u, 0u);
            p[u] = ok ? s_sc[i] * inv_l : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float vf[8];
            unpack8(vr[u], vf);
#pragma unroll
            for (int j = 0; j < 8; j++) o[j] = fmaf(p[u], vf[j], o[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++) s_o[warp][lane * 8 + j] = o[j];
    __syncthreads();
    if (t >= ATT_D) return;
    float acc = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) acc += s_o[w][t];

    const float a = round_f16(acc);
    const float gt = __half2float(gate[(size_t)h * ATT_D + t]);
    const float sg = round_f16(1.0f / (1.0f + expf(-gt)));
    out[(size_t)h * ATT_D + t] = __float2half(a * sg);
}

// Decode: one token, length read from device memory.
__global__ void __launch_bounds__(ATT_THREADS)
attn_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ keys,
                   const __half* __restrict__ values, const long long* __restrict__ cum_len,
                   const __half* __restrict__ gate, __half* __restrict__ out, int max_len,
                   int gqa, float scale) {
    pdl_prologue();
    PDL_FRESH(q); PDL_FRESH(keys); PDL_FRESH(values); PDL_FRESH(cum_len); PDL_FRESH(gate); PDL_FRESH(out);
    long long L64 = *cum_len;
    if (L64 > max_len) L64 = max_len;  // never index past the cache
    if (L64 < 0) L64 = 0;
    attn_one_query(q, keys, values, (int)L64, gate, out, max_len, gqa, scale);
}

// ---------------------------------------------------------------------------------------------
// Gated DeltaNet decode step (head dim 128, conv kernel 4; 16 key / 48 value heads in the full
// model, fewer on a tensor-parallel shard).
// Kernel 1: causal conv1d update + silu per channel -> scratch (fp32 holding fp16-rounded values).
// Kernel 2: one CTA per value head, 16 warps; a warp owns 8 state rows (one row = 128 fp32 =
//           one float4 per lane, so every state access is a coalesced 512-byte row).
// ---------------------------------------------------------------------------------------------
#define DN_DK 128
#define DN_NVH 48
#define DN_KEY_DIM 2048
#define DN_CONV_DIM 10240
#define DN_REC_THREADS 512

__device__ __forceinline__ float softplus_f(float x) { return (x > 20.0f) ? x : log1pf(expf(x)); }

__global__ void __launch_bounds__(256)
dn_conv_kernel(const __half* __restrict__ mixed, const __half* __restrict__ conv_w,
               __half* __restrict__ conv_state, float* __restrict__ scratch, int conv_dim) {
    // Wait first, then let the next kernel start: dn_rec_kernel reads the recurrent state before
    // its own wait, which is safe only once everything before this kernel — possibly a
    // dn_rec_kernel on the same state, when two tokens are processed back to back — has finished.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    PDL_FRESH(mixed); PDL_FRESH(conv_state); PDL_FRESH(scratch);
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= conv_dim) return;
    // state and weights of a channel are 4 consecutive halves: one 8-byte load each
    const uint2 sv = *reinterpret_cast<const uint2*>(conv_state + (size_t)c * 4);
    const uint2 wv = *reinterpret_cast<const uint2*>(conv_w + (size_t)c * 4);
    const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x);
    const __half2 s23 = *reinterpret_cast<const __half2*>(&sv.y);
    const __half2 w01 = *reinterpret_cast<const __half2*>(&wv.x);
    const __half2 w23 = *reinterpret_cast<const __half2*>(&wv.y);
    const __half x = mixed[c];
    const float s1 = __high2float(s01), s2 = __low2float(s23), s3 = __high2float(s23);
    // window [s1, s2, s3, x]; the sum is evaluated left to right with fused multiply-adds
    float acc = __low2float(w01) * s1;
    acc = fmaf(__high2float(w01), s2, acc);
    acc = fmaf(__low2float(w23), s3, acc);
    acc = fmaf(__high2float(w23), __half2float(x), acc);
    scratch[c] = round_f16(silu_f(acc));
    uint2 ns;
    const __half2 n01 = __halves2half2(__high2half(s01), __low2half(s23));
    const __half2 n23 = __halves2half2(__high2half(s23), x);
    ns.x = *reinterpret_cast<const uint32_t*>(&n01);
    ns.y = *reinterpret_cast<const uint32_t*>(&n23);
    *reinterpret_cast<uint2*>(conv_state + (size_t)c * 4) = ns;
}

__global__ void __launch_bounds__(DN_REC_THREADS)
dn_rec_kernel(const __half* __restrict__ z_in, const __half* __restrict__ b_in,
              const __half* __restrict__ a_in, const __half* __restrict__ A_log,
              const __half* __restrict__ dt_bias, const __half* __restrict__ norm_w,
              const float* __restrict__ scratch, float* __restrict__ state,
              __half* __restrict__ out, float rms_eps, int key_dim, int rep) {
    __shared__ float s_o[DN_DK];
    __shared__ float s_red[8];
    const int h = blockIdx.x, kh = h / rep;  // value head h reads key head h / rep
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    // The recurrent state was last written by this kernel's own launch of the previous step, so
    // its 64 KB per head are requested before waiting for the previous kernel in the stream;
    // everything that kernel produces (conv output, z, b, a) is read after the wait.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    float* Sbase = state + ((size_t)h * DN_DK + (size_t)warp * 8) * DN_DK + lane * 4;
    float4 S[8];
#pragma unroll
    for (int r = 0; r < 8; r++) S[r] = *reinterpret_cast<const float4*>(Sbase + (size_t)r * DN_DK);
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    PDL_FRESH(z_in); PDL_FRESH(b_in); PDL_FRESH(a_in); PDL_FRESH(scratch); PDL_FRESH(out);

    const float beta = round_f16(1.0f / (1.0f + expf(-__half2float(b_in[h]))));
    const float gdec = -expf(__half2float(A_log[h])) *
                       softplus_f(__half2float(a_in[h]) + __half2float(dt_bias[h]));
    const float eg = expf(gdec);

    // every warp normalises q and k itself: lane owns dims 4*lane .. 4*lane+3
    float4 qv = *reinterpret_cast<const float4*>(scratch + kh * DN_DK + lane * 4);
    float4 kv = *reinterpret_cast<const float4*>(scratch + key_dim + kh * DN_DK + lane * 4);
    const float qss = warp_sum(qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w);
    const float kss = warp_sum(kv.x * kv.x + kv.y * kv.y + kv.z * kv.z + kv.w * kv.w);
    const float inv_q = rsqrtf(qss + 1e-6f) * 0.08838834764831845f;
    const float inv_k = rsqrtf(kss + 1e-6f);
    qv.x *= inv_q; qv.y *= inv_q; qv.z *= inv_q; qv.w *= inv_q;
    kv.x *= inv_k; kv.y *= inv_k; kv.z *= inv_k; kv.w *= inv_k;

    // rows j = warp*8 .. warp*8+7 of S_t[h][j][:]
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const int j = warp * 8 + r;
        S[r].x *= eg; S[r].y *= eg; S[r].z *= eg; S[r].w *= eg;
        float kvp = S[r].x * kv.x;
        kvp = fmaf(S[r].y, kv.y, kvp);
        kvp = fmaf(S[r].z, kv.z, kvp);
        kvp = fmaf(S[r].w, kv.w, kvp);
        kvp = warp_sum(kvp);
        const float v_j = scratch[key_dim * 2 + h * DN_DK + j];
        const float delta = (v_j - kvp) * beta;
        S[r].x = fmaf(kv.x, delta, S[r].x);
        S[r].y = fmaf(kv.y, delta, S[r].y);
        S[r].z = fmaf(kv.z, delta, S[r].z);
        S[r].w = fmaf(kv.w, delta, S[r].w);
        *reinterpret_cast<float4*>(Sbase + (size_t)r * DN_DK) = S[r];
        float o = S[r].x * qv.x;
        o = fmaf(S[r].y, qv.y, o);
        o = fmaf(S[r].z, qv.z, o);
        o = fmaf(S[r].w, qv.w, o);
        o = warp_sum(o);
        if (lane == 0) s_o[j] = round_f16(o);
    }
    __syncthreads();
    // RMSNormGated over the head's 128 outputs, then * silu(z)
    if (warp < 4) {
        const int j = t;  // 0..127
        const float o = s_o[j];
        float ss = warp_sum(o * o);
        if (lane == 0) s_red[warp] = ss;
    }
    __syncthreads();
    if (t < DN_DK) {
        const float var_mean = ((s_red[0] + s_red[1]) + (s_red[2] + s_red[3])) / (float)DN_DK;
        const float o = s_o[t];
        const float xn = o * rsqrtf(var_mean + rms_eps);
        const __half hw = __hmul(__float2half(xn), norm_w[t]);
        const float res = __half2float(hw) * silu_f(__half2float(z_in[(size_t)h * DN_DK + t]));
        out[(size_t)h * DN_DK + t] = __float2half(res);
    }
}

// Decode attention split over the keys (flash-decoding): ATS_SPLIT CTAs per query head, each
// taking every ATS_SPLIT-th block of ATS_WARPS keys.  A warp requests up to ATS_ROWS key rows AND
// the matching value rows at once (values do not depend on the scores), so a context of up to
// ATS_SPLIT * ATS_WARPS * ATS_ROWS = 768 keys costs one memory round trip instead of one per
// four keys; longer contexts loop.  Each warp keeps a running (max, sum, weighted values); warps
// combine through shared memory, CTAs through a scratch buffer in global memory, and the CTA
// that arrives last at the head's counter (in whatever order the CTAs finish, the partials are
// combined in split order, so the result is deterministic) applies 1/sum, rounds to fp16 and
// multiplies by sigmoid(gate) as attn_one_query does.  Scores use the same fma chain; the
// softmax is rescaled per part, so results can differ from attn_one_query in the last fp32 bit
// before the fp16 rounding.
#define ATS_SPLIT 8
#define ATS_WARPS 16
#define ATS_ROWS 6
#define ATS_PART (ATT_D + 4)    // floats per partial: 256 weighted values, max, sum, padding

__global__ void __launch_bounds__(ATS_WARPS * 32)
attn_decode_split_kernel(const __half* __restrict__ q, const __half* __restrict__ keys,
                         const __half* __restrict__ values, const long long* __restrict__ cum_len,
                         const __half* __restrict__ gate, __half* __restrict__ out,
                         float* __restrict__ part, unsigned int* __restrict__ counters,
                         int max_len, int gqa, float scale) {
    pdl_prologue();
    PDL_FRESH(q); PDL_FRESH(keys); PDL_FRESH(values); PDL_FRESH(cum_len); PDL_FRESH(gate); PDL_FRESH(out);
    PDL_FRESH(part); PDL_FRESH(counters);
    __shared__ float s_part[ATS_WARPS][ATS_PART];
    __shared__ unsigned int s_last;
    const int h = blockIdx.x, sp = blockIdx.y, kv = h / gqa;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    long long L64 = *cum_len;
    if (L64 > max_len) L64 = max_len;
    if (L64 < 0) L64 = 0;
    const int L = (int)L64;

    float qf[8];
    unpack8(*reinterpret_cast<const uint4*>(q + (size_t)h * ATT_D + lane * 8), qf);
    const __half* kbase = keys + (size_t)kv * (size_t)max_len * ATT_D + lane * 8;
    const __half* vbase = values + (size_t)kv * (size_t)max_len * ATT_D + lane * 8;
    float m = -3.4e38f, l = 0.0f;
    float o[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    // key i belongs to split (i / ATS_WARPS) % ATS_SPLIT and warp i % ATS_WARPS
    const int stride = ATS_SPLIT * ATS_WARPS;
    for (int i0 = sp * ATS_WARPS + warp; i0 < L; i0 += stride * ATS_ROWS) {
        uint4 kr[ATS_ROWS], vr[ATS_ROWS];
#pragma unroll
        for (int u = 0; u < ATS_ROWS; u++) {
            const int i = i0 + u * stride;
            const bool ok = i < L;
            kr[u] = ok ? *reinterpret_cast<const uint4*>(kbase + (size_t)i * ATT_D)
                       : make_uint4(0u, 0u, 0u, 0u);
            vr[u] = ok ? *reinterpret_cast<const uint4*>(vbase + (size_t)i * ATT_D)
                       : make_uint4(0u, 0u, 0u, 0u);
        }
        float sc[ATS_ROWS];
        float mb = m;
#pragma unroll
        for (int u = 0; u < ATS_ROWS; u++) {
            float kf[8];
            unpack8(kr[u], kf);
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) acc = fmaf(qf[j], kf[j], acc);
            acc = warp_sum(acc) * scale;
            sc[u] = (i0 + u * stride < L) ? acc : -3.4e38f;
            mb = fmaxf(mb, sc[u]);
        }
        const float corr = expf(m - mb);          // 0 on the first batch (m = -3.4e38)
        l *= corr;
#pragma unroll
        for (int j = 0; j < 8; j++) o[j] *= corr;
        m = mb;
#pragma unroll
        for (int u = 0; u < ATS_ROWS; u++) {
            const float p = (i0 + u * stride < L) ? expf(sc[u] - m) : 0.0f;
            l += p;
            float vf[8];
            unpack8(vr[u], vf);
#pragma unroll
            for (int j = 0; j < 8; j++) o[j] = fmaf(p, vf[j], o[j]);
        }
    }
    // ---- warps -> CTA partial ----
#pragma unroll
    for (int j = 0; j < 8; j++) s_part[warp][lane * 8 + j] = o[j];
    if (lane == 0) {
        s_part[warp][ATT_D] = m;
        s_part[warp][ATT_D + 1] = l;
    }
    __syncthreads();
    float* mine = part + ((size_t)h * ATS_SPLIT + sp) * ATS_PART;
    if (t < ATT_D) {
        float M = -3.4e38f;
#pragma unroll
        for (int w = 0; w < ATS_WARPS; w++) M = fmaxf(M, s_part[w][ATT_D]);
        float acc = 0.0f, ls = 0.0f;
#pragma unroll
        for (int w = 0; w < ATS_WARPS; w++) {
            const float f = expf(s_part[w][ATT_D] - M);     // warps without keys: exp(-huge) = 0
            acc = fmaf(s_part[w][t], f, acc);
            ls = fmaf(s_part[w][ATT_D + 1], f, ls);
        }
        mine[t] = acc;
        if (t == 0) {
            mine[ATT_D] = M;
            mine[ATT_D + 1] = ls;
        }
    }
    // ---- CTAs -> head: the last CTA to arrive combines the parts in split order ----
    __threadfence();
    __syncthreads();
    if (t == 0) {
        const unsigned int prev = atomicAdd(counters + h, 1u);
        s_last = (prev == ATS_SPLIT - 1) ? 1u : 0u;
        if (s_last) counters[h] = 0u;                       // ready for the next launch
    }
    __syncthreads();
    if (!s_last || t >= ATT_D) return;
    __threadfence();
    const float* ph = part + (size_t)h * ATS_SPLIT * ATS_PART;
    float M = -3.4e38f;
#pragma unroll
    for (int s = 0; s < ATS_SPLIT; s++) M = fmaxf(M, __ldcg(ph + s * ATS_PART + ATT_D));
    float acc = 0.0f, ls = 0.0f;
#pragma unroll
    for (int s = 0; s < ATS_SPLIT; s++) {
        const float f = expf(__ldcg(ph + s * ATS_PART + ATT_D) - M);
        acc = fmaf(__ldcg(ph + s * ATS_PART + t), f, acc);
        ls = fmaf(__ldcg(ph + s * ATS_PART + ATT_D + 1), f, ls);
    }
    const float a = round_f16(acc * (1.0f / ls));
    const float gt = __half2float(gate[(size_t)h * ATT_D + t]);
    const float sg = round_f16(1.0f / (1.0f + expf(-gt)));
    out[(size_t)h * ATT_D + t] = __float2half(a * sg);
}

// Prefill attention for ATT_G consecutive tokens of one query head per CTA: the tokens share
// every key and value row they load (token g of the group sees L0 + g rows).  Per token the
// arithmetic and its order are those of attn_one_query — same key-to-warp assignment, same
// reduction trees — so a chunk gives bit-identical outputs to token-by-token decode.
#define ATT_G 4
__global__ void __launch_bounds__(ATT_THREADS)
attn_prefill_group_kernel(const __half* __restrict__ q, const __half* __restrict__ keys,
                          const __half* __restrict__ values, int len0, int n_tokens,
                          const __half* __restrict__ gate, __half* __restrict__ out, int max_len,
                          int gqa, float scale, int lcap) {
    pdl_prologue();
    PDL_FRESH(q); PDL_FRESH(keys); PDL_FRESH(values); PDL_FRESH(gate); PDL_FRESH(out);
    extern __shared__ float s_sc[];                 // [ATT_G][lcap]
    __shared__ float s_q[ATT_G][ATT_D];
    __shared__ float s_red[ATT_G][ATT_WARPS];
    __shared__ float s_bcast[ATT_G];
    __shared__ float s_o[ATT_WARPS][ATT_D];
    const int h = blockIdx.x, kv = h / gqa, hq = gridDim.x;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int tok0 = blockIdx.y * ATT_G;
    int Lg[ATT_G];
#pragma unroll
    for (int g = 0; g < ATT_G; g++) {
        const int tok = tok0 + g;
        int L = (tok < n_tokens) ? len0 + tok : 0;   // 0 rows: the token does not exist
        Lg[g] = min(L, max_len);
    }
    int Lmax = 0;
#pragma unroll
    for (int g = 0; g < ATT_G; g++) Lmax = max(Lmax, Lg[g]);
    if (t < ATT_D) {
#pragma unroll
        for (int g = 0; g < ATT_G; g++)
            s_q[g][t] = (Lg[g] > 0)
                            ? __half2float(q[((size_t)(tok0 + g) * hq + h) * ATT_D + t]) : 0.0f;
    }
    __syncthreads();

    const __half* kbase = keys + (size_t)kv * (size_t)max_len * ATT_D + lane * 8;
    float m[ATT_G];
#pragma unroll
    for (int g = 0; g < ATT_G; g++) m[g] = -3.4e38f;
    for (int i0 = warp; i0 < Lmax; i0 += ATT_WARPS * 2) {
        uint4 kr[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int i = i0 + u * ATT_WARPS;
            kr[u] = (i < Lmax) ? *reinterpret_cast<const uint4*>(kbase + (size_t)i * ATT_D)
                               : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int i = i0 + u * ATT_WARPS;
            float kf[8];
            unpack8(kr[u], kf);
#pragma unroll
            for (int g = 0; g < ATT_G; g++) {
                const float4 qa = *reinterpret_cast<const float4*>(&s_q[g][lane * 8]);
                const float4 qb = *reinterpret_cast<const float4*>(&s_q[g][lane * 8 + 4]);
                float acc = 0.0f;
                acc = fmaf(qa.x, kf[0], acc); acc = fmaf(qa.y, kf[1], acc);
                acc = fmaf(qa.z, kf[2], acc); acc = fmaf(qa.w, kf[3], acc);
                acc = fmaf(qb.x, kf[4], acc); acc = fmaf(qb.y, kf[5], acc);
                acc = fmaf(qb.z, kf[6], acc); acc = fmaf(qb.w, kf[7], acc);
                acc = warp_sum(acc) * scale;
                if (i < Lg[g]) {
                    if (lane == 0) s_sc[(size_t)g * lcap + i] = acc;
                    m[g] = fmaxf(m[g], acc);
                }
            }
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < ATT_G; g++) s_red[g][warp] = m[g];
    }
    __syncthreads();
    if (warp < ATT_G) {
        float v = s_red[warp][lane];                // ATT_WARPS == 32 values per token
        v = warp_max(v);
        if (lane == 0) s_bcast[warp] = v;
    }
    __syncthreads();
    float l[ATT_G];
#pragma unroll
    for (int g = 0; g < ATT_G; g++) {
        const float mg = s_bcast[g];
        float a = 0.0f;
        for (int i = t; i < Lg[g]; i += ATT_THREADS) {
            const float e = expf(s_sc[(size_t)g * lcap + i] - mg);
            s_sc[(size_t)g * lcap + i] = e;
            a += e;
        }
        l[g] = warp_sum(a);
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < ATT_G; g++) s_red[g][warp] = l[g];
    }
    __syncthreads();
    if (warp < ATT_G) {
        float v = s_red[warp][lane];
        v = warp_sum(v);
        if (lane == 0) s_bcast[warp] = 1.0f / v;
    }
    __syncthreads();
    float inv_l[ATT_G];
#pragma unroll
    for (int g = 0; g < ATT_G; g++) inv_l[g] = s_bcast[g];

    const __half* vbase = values + (size_t)kv * (size_t)max_len * ATT_D + lane * 8;
    float o[ATT_G][8];
#pragma unroll
    for (int g = 0; g < ATT_G; g++)
#pragma unroll
        for (int j = 0; j < 8; j++) o[g][j] = 0.0f;
    for (int i0 = warp; i0 < Lmax; i0 += ATT_WARPS * 2) {
        uint4 vr[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int i = i0 + u * ATT_WARPS;
            vr[u] = (i < Lmax) ? *reinterpret_cast<const uint4*>(vbase + (size_t)i * ATT_D)
                               : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int i = i0 + u * ATT_WARPS;
            float vf[8];
            unpack8(vr[u], vf);
#pragma unroll
            for (int g = 0; g < ATT_G; g++) {
                const float p = (i < Lg[g]) ? s_sc[(size_t)g * lcap + i] * inv_l[g] : 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j++) o[g][j] = fmaf(p, vf[j], o[g][j]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < ATT_G; g++) {
        __syncthreads();                            // s_o free (first round: nothing pending)
#pragma unroll
        for (int j = 0; j < 8; j++) s_o[warp][lane * 8 + j] = o[g][j];
        __syncthreads();
        if (t < ATT_D && Lg[g] > 0) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; w++) acc += s_o[w][t];
            const size_t idx = ((size_t)(tok0 + g) * hq + h) * ATT_D + t;
            const float a = round_f16(acc);
            const float gt = __half2float(gate[idx]);
            const float sg = round_f16(1.0f / (1.0f + expf(-gt)));
            out[idx] = __float2half(a * sg);
        }
    }
}

}  // namespace nvfp4

extern "C" {

int launch_rmsnorm(const void* x, long long row_stride, const void* w1, void* out, int rows, int n,
                   float eps, void* stream) {
    if (rows <= 0 || n <= 0) return -1;
    if (!x || !w1 || !out) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (n >= 2048)
        e = nvfp4::launch_pdl(nvfp4::rmsnorm_kernel<512>, dim3(rows), dim3(512), 0, st,
                              (const __half*)x, row_stride, (const float*)w1, (__half*)out, n, eps);
    else
        e = nvfp4::launch_pdl(nvfp4::rmsnorm_kernel<64>, dim3(rows), dim3(64), 0, st,
                              (const __half*)x, row_stride, (const float*)w1, (__half*)out, n, eps);
    return (e == cudaSuccess) ? 0 : (int)e;
}

int launch_rope_qk(const void* q, const void* k, const void* cs, const void* sn, void* q_out,
                   void* k_out, int hq, int hkv, void* stream) {
    if (hq < 0 || hkv < 0 || hq + hkv <= 0) return -1;
    if (!cs || !sn || (hq > 0 && (!q || !q_out)) || (hkv > 0 && (!k || !k_out))) return -1;
    const cudaError_t e = nvfp4::launch_pdl(
        nvfp4::rope_qk_kernel, dim3(hq + hkv), dim3(128), 0, (cudaStream_t)stream, (const __half*)q,
        (const __half*)k, (const __half*)cs, (const __half*)sn, (__half*)q_out, (__half*)k_out, hq);
    return e == cudaSuccess ? 0 : -2;
}

int launch_silu_mul(const void* g, const void* u, void* out, int n, void* stream) {
    if (n <= 0 || !g || !u || !out) return -1;
    const cudaError_t e =
        nvfp4::launch_pdl(nvfp4::silu_mul_kernel, dim3((n + 255) / 256), dim3(256), 0,
                          (cudaStream_t)stream, (const __half*)g, (const __half*)u, (__half*)out, n);
    return e == cudaSuccess ? 0 : -2;
}

// Heads are the 27B model's: 24 query heads, 4 KV heads, head dim 256.  max_len is the cache's
// allocated length and may be any value whose fp32 score buffer fits in shared memory
// (max_len <= 47104); larger values return -2, as the reference does for an unsupported length.
static int attn_decode_launch(const void* q, const void* keys, const void* values,
                              const void* cum_len, const void* gate, void* out, int max_len,
                              int hq, int hkv, float scale, void* stream) {
    static bool smem_opt_in[nvfp4::NVFP4_MAX_DEVICES] = {false};
    const int dev = nvfp4::current_device_index();
    if (max_len <= 0 || max_len > 47104) return -2;
    if (!q || !keys || !values || !cum_len || !gate || !out) return -2;
    if (hq <= 0 || hkv <= 0 || hq % hkv != 0) return -2;
    const size_t smem = (size_t)max_len * sizeof(float);
    if (!smem_opt_in[dev]) {
        // one-time (per device) opt-in to the large dynamic shared memory carve-out (a host-side attribute,
        // not a stream operation)
        if (cudaFuncSetAttribute(nvfp4::attn_decode_kernel,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(47104 * sizeof(float))) != cudaSuccess)
            return -2;
        smem_opt_in[dev] = true;
    }
    const cudaError_t e = nvfp4::launch_pdl(
        nvfp4::attn_decode_kernel, dim3(hq), dim3(ATT_THREADS), smem, (cudaStream_t)stream,
        (const __half*)q, (const __half*)keys, (const __half*)values, (const long long*)cum_len,
        (const __half*)gate, (__half*)out, max_len, hq / hkv, scale);
    return (e == cudaSuccess) ? 0 : (int)e;
}

// Causal attention of a prefill chunk with the decode kernel's arithmetic: token i of the chunk
// (i < n_tokens) attends to cache rows [0, len0 + i), which must already hold the chunk's own
// keys and values.  q, gate, out: token-major [n_tokens][hq * 256].  Grid (hq, n_tokens).
int launch_attn_prefill(const void* q, const void* keys, const void* values, int len0,
                        int n_tokens, const void* gate, void* out, int max_len, int hq, int hkv,
                        float scale, void* stream) {
    static int smem_set[nvfp4::NVFP4_MAX_DEVICES] = {0};
    const int dev = nvfp4::current_device_index();
    if (max_len <= 0 || max_len > 47104 || n_tokens <= 0 || n_tokens > 65535) return -2;
    if (len0 < 1 || len0 + n_tokens - 1 > max_len) return -2;
    if (!q || !keys || !values || !gate || !out) return -2;
    if (hq <= 0 || hkv <= 0 || hq % hkv != 0) return -2;
    const int lcap = len0 + n_tokens - 1;
    const int smem = ATT_G * lcap * (int)sizeof(float);
    if (smem > 150 * 1024) return -2;
    if (smem > 8 * 1024 && smem > smem_set[dev]) {
        if (cudaFuncSetAttribute(nvfp4::attn_prefill_group_kernel,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return -2;
        smem_set[dev] = smem;
    }
    const cudaError_t e = nvfp4::launch_pdl(
        nvfp4::attn_prefill_group_kernel, dim3(hq, (n_tokens + ATT_G - 1) / ATT_G),
        dim3(ATT_THREADS), (size_t)smem, (cudaStream_t)stream, (const __half*)q,
        (const __half*)keys, (const __half*)values, len0, n_tokens, (const __half*)gate,
        (__half*)out, max_len, hq / hkv, scale, lcap);
    return (e == cudaSuccess) ? 0 : (int)e;
}

// Bytes of scratch launch_attn_decode_split needs for hq query heads (partials + one counter per
// head); the counters (the last hq * 4 bytes ... see the launcher) must be zero before first use.
long long nvfp4_attn_split_scratch_bytes(int hq) {
    if (hq <= 0) return -1;
    return (long long)hq * ATS_SPLIT * ATS_PART * 4 + (long long)hq * 4;
}

// launch_attn_decode_heads with the keys split over eight CTAs per head.  scratch: device buffer
// of nvfp4_attn_split_scratch_bytes(hq) bytes, 16-byte aligned, zeroed once by the caller (the
// kernel leaves its counters at zero).  Calls that share a scratch buffer must not overlap.
// 0; -2 bad arguments; else the launch error.
int launch_attn_decode_split(const void* q, const void* keys, const void* values,
                             const void* cum_len, const void* gate, void* out, void* scratch,
                             int max_len, int hq, int hkv, float scale, void* stream) {
    if (max_len <= 0 || !q || !keys || !values || !cum_len || !gate || !out || !scratch) return -2;
    if (hq <= 0 || hkv <= 0 || hq % hkv != 0 || ((uintptr_t)scratch & 15)) return -2;
    float* part = (float*)scratch;
    unsigned int* counters = (unsigned int*)(part + (size_t)hq * ATS_SPLIT * ATS_PART);
    const cudaError_t e = nvfp4::launch_pdl(
        nvfp4::attn_decode_split_kernel, dim3(hq, ATS_SPLIT), dim3(ATS_WARPS * 32), 0,
        (cudaStream_t)stream, (const __half*)q, (const __half*)keys, (const __half*)values,
        (const long long*)cum_len, (const __half*)gate, (__half*)out, part, counters, max_len,
        hq / hkv, scale);
    return (e == cudaSuccess) ? 0 : (int)e;
}

int launch_attn_decode(const void* q, const void* keys, const void* values, const void* cum_len,
                       const void* gate, void* out, int max_len, float scale, void* stream) {
    return attn_decode_launch(q, keys, values, cum_len, gate, out, max_len, 24, 4, scale, stream);
}

// The same kernel for a tensor-parallel shard or a smaller model: hq query heads, hkv KV heads
// (hq a multiple of hkv), head dim 256.
int launch_attn_decode_heads(const void* q, const void* keys, const void* values,
                             const void* cum_len, const void* gate, void* out, int max_len, int hq,
                             int hkv, float scale, void* stream) {
    return attn_decode_launch(q, keys, values, cum_len, gate, out, max_len, hq, hkv, scale, stream);
}

static int dn_fused_launch(const void* mixed, const void* z_in, const void* b_in, const void* a_in,
                           const void* conv_w, void* conv_state, const void* A_log,
                           const void* dt_bias, const void* norm_w, void* state, void* scratch,
                           void* out, int n_kheads, int n_vheads, float rms_eps, void* stream) {
    if (!mixed || !z_in || !b_in || !a_in || !conv_w || !conv_state || !A_log || !dt_bias ||
        !norm_w || !state || !scratch || !out)
        return -1;
    if (n_kheads <= 0 || n_vheads <= 0 || n_vheads % n_kheads != 0) return -1;
    const int key_dim = n_kheads * DN_DK;
    const int conv_dim = 2 * key_dim + n_vheads * DN_DK;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = nvfp4::launch_pdl(nvfp4::dn_conv_kernel, dim3((conv_dim + 255) / 256), dim3(256),
                                      0, s, (const __half*)mixed, (const __half*)conv_w,
                                      (__half*)conv_state, (float*)scratch, conv_dim);
    if (e != cudaSuccess) {
        fprintf(stderr, "dn_conv launch: %s\n", cudaGetErrorString(e));
        return -1;
    }
    e = nvfp4::launch_pdl(nvfp4::dn_rec_kernel, dim3(n_vheads), dim3(DN_REC_THREADS), 0, s,
                          (const __half*)z_in, (const __half*)b_in, (const __half*)a_in,
                          (const __half*)A_log, (const __half*)dt_bias, (const __half*)norm_w,
                          (const float*)scratch, (float*)state, (__half*)out, rms_eps, key_dim,
                          n_vheads / n_kheads);
    if (e != cudaSuccess) {
        fprintf(stderr, "dn_rec launch: %s\n", cudaGetErrorString(e));
        return -1;
    }
    return 0;
}

int launch_dn_fused(const void* mixed, const void* z_in, const void* b_in, const void* a_in,
                    const void* conv_w, void* conv_state, const void* A_log, const void* dt_bias,
                    const void* norm_w, void* state, void* scratch, void* out, float rms_eps,
                    void* stream) {
    return dn_fused_launch(mixed, z_in, b_in, a_in, conv_w, conv_state, A_log, dt_bias, norm_w,
                           state, scratch, out, DN_KEY_DIM / DN_DK, DN_NVH, rms_eps, stream);
}

// Same step for a tensor-parallel shard that holds n_kheads key heads and n_vheads value heads
// (n_vheads a multiple of n_kheads): mixed is [q n_k*128 | k n_k*128 | v n_v*128], every other
// buffer shrinks accordingly, scratch holds (2 n_k + n_v) * 128 floats.
int launch_dn_fused_heads(const void* mixed, const void* z_in, const void* b_in, const void* a_in,
                          const void* conv_w, void* conv_state, const void* A_log,
                          const void* dt_bias, const void* norm_w, void* state, void* scratch,
                          void* out, int n_kheads, int n_vheads, float rms_eps, void* stream) {
    return dn_fused_launch(mixed, z_in, b_in, a_in, conv_w, conv_state, A_log, dt_bias, norm_w,
                           state, scratch, out, n_kheads, n_vheads, rms_eps, stream);
}

// ---------------------------------------------------------------------------------------------
// DeltaNet step for callers that cannot allocate device memory.
//
// The step needs a small workspace between its two kernels (the conv+silu result, one float per
// conv channel).  launch_dn_fused makes the caller provide it.  Some callers cannot: a host loop
// that has already handed every byte of device memory to another allocator, a plug-in that is
// only given its input and output buffers, or code that is entered while the stream is being
// captured (cudaMalloc synchronises the device and is not permitted there).  For them the
// workspace lives in the library itself: a file-scope device array of
// NVFP4_DN_NOALLOC_MAX_CHANNELS floats (40 KB), which every GPU that loads the library keeps
// until the process exits.
//
// Host code may not hand the array's name to a kernel: in host code the name is only a handle
// for the runtime, not a device address.  The address is obtained with cudaGetSymbolAddress,
// once per device, with that device current, and cached.  That look-up happens on the first
// call on each device, so make the first call on a device outside any stream capture.
//
// All calls on one device share the workspace.  Nothing in it has to start at zero (the first
// kernel writes every element the second one reads), so it is never cleared; but two calls that
// run on the GPU at the same time (different streams, or graph branches) would overwrite each
// other's intermediate values: keep calls on one device ordered.
// The function calls no cudaMalloc, cudaFree or any other allocating routine.
// ---------------------------------------------------------------------------------------------
#define NVFP4_DN_NOALLOC_MAX_CHANNELS 10240
#define NVFP4_DN_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) float g_dn_noalloc_scratch[NVFP4_DN_NOALLOC_MAX_CHANNELS];
static float* g_dn_noalloc_addr[NVFP4_DN_NOALLOC_MAX_DEVICES] = {};

int launch_dn_fused_noalloc(const void* mixed, const void* z_in, const void* b_in,
                            const void* a_in, const void* conv_w, void* conv_state,
                            const void* A_log, const void* dt_bias, const void* norm_w,
                            void* state, void* out, int n_kheads, int n_vheads, float rms_eps,
                            void* stream) {
    if (n_kheads <= 0 || n_vheads <= 0 || n_vheads % n_kheads != 0) return -1;
    const long long channels = (2LL * n_kheads + n_vheads) * DN_DK;
    if (channels > NVFP4_DN_NOALLOC_MAX_CHANNELS) {
        fprintf(stderr,
                "launch_dn_fused_noalloc: %lld conv channels (%d key + %d value heads) exceed the "
                "built-in workspace of %d; use launch_dn_fused_heads with your own scratch\n",
                channels, n_kheads, n_vheads, NVFP4_DN_NOALLOC_MAX_CHANNELS);
        return -2;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NVFP4_DN_NOALLOC_MAX_DEVICES) {
        fprintf(stderr, "launch_dn_fused_noalloc: no usable current device\n");
        return -1;
    }
    float* scratch = g_dn_noalloc_addr[dev];
    if (scratch == nullptr) {
        const cudaError_t e = cudaGetSymbolAddress((void**)&scratch, g_dn_noalloc_scratch);
        if (e != cudaSuccess || scratch == nullptr) {
            fprintf(stderr, "launch_dn_fused_noalloc: cudaGetSymbolAddress: %s\n",
                    cudaGetErrorString(e));
            return -1;
        }
        g_dn_noalloc_addr[dev] = scratch;
    }
    return dn_fused_launch(mixed, z_in, b_in, a_in, conv_w, conv_state, A_log, dt_bias, norm_w,
                           state, scratch, out, n_kheads, n_vheads, rms_eps, stream);
}

}  // extern "C"

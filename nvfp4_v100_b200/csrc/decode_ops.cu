// Small kernels that glue one decode step together on the device, so that a whole step — from
// the previous token id to the next one — is a fixed sequence of launches that a CUDA graph can
// replay without host work in between.
//
// In the reference these pieces are PyTorch operators inside the captured model forward
// (pipeline/_qwen38_infer.py:679-685: the forward, logits[:, -1].argmax, static_pos.add_(1)) and
// a host-side embedding gather before each replay (:714-716).  Position-dependent work reads the
// position from device memory, as the reference's attention kernel does with cum_len
// (kernels/nvfp4_attn_decode.cu:33,43).
#include <cstdio>

#include "common.cuh"

namespace nvfp4 {

// out[0..hidden) = table[tok][0..hidden), tok read from device memory.
__global__ void __launch_bounds__(256)
embed_gather_kernel(const __half* __restrict__ table, const long long* __restrict__ tok,
                    __half* __restrict__ out, int hidden, long long vocab) {
    pdl_prologue();
    PDL_FRESH(table); PDL_FRESH(tok); PDL_FRESH(out);
    long long id = *tok;
    if (id < 0) id = 0;
    if (id >= vocab) id = vocab - 1;
    const int i = (blockIdx.x * 256 + threadIdx.x) * 8;
    if (i + 8 <= hidden) {
        *reinterpret_cast<uint4*>(out + i) =
            *reinterpret_cast<const uint4*>(table + (size_t)id * hidden + i);
    } else {
        for (int j = i; j < hidden; j++) out[j] = table[(size_t)id * hidden + j];
    }
}

// Everything between the q/k/v projection and the attention kernel, one CTA per head:
//   query head h : q = rmsnorm(qkv[h*512 .. +256]) with q_w1, RoPE at *pos -> q_out[h];
//                  gate_out[h] = qkv[h*512+256 .. +256]   (the projection emits [q | gate] per head)
//   key head j   : k = rmsnorm(k_j) with k_w1, RoPE at *pos -> keys[j][*pos]
//   value head j : values[j][*pos] = v_j
// RMSNorm and RoPE use exactly the arithmetic of rmsnorm_kernel and rope_qk_kernel, including the
// fp16 rounding between them.
__device__ __forceinline__ void attn_prep_one_token(
    const __half* __restrict__ qkv, const float* __restrict__ q_w1, const float* __restrict__ k_w1,
    const __half* __restrict__ cos_tab, const __half* __restrict__ sin_tab, long long pos,
    __half* __restrict__ q_out, __half* __restrict__ gate_out, __half* __restrict__ keys,
    __half* __restrict__ values, int hq, int hkv, int max_len, float eps) {
    __shared__ float s_red[8];
    __shared__ float s_n[256];
    const int b = blockIdx.x, d = threadIdx.x, lane = d & 31, warp = d >> 5;
    if (pos < 0) pos = 0;
    if (pos >= max_len) pos = max_len - 1;  // never index past the cache or the tables
    const __half* kbase = qkv + (size_t)hq * 512;
    const __half* vbase = kbase + (size_t)hkv * 256;
    if (b >= hq + hkv) {  // value head: plain copy into the cache
        const int j = b - hq - hkv;
        values[((size_t)j * max_len + pos) * 256 + d] = vbase[(size_t)j * 256 + d];
        return;
    }
    const bool is_q = b < hq;
    const __half* src = is_q ? qkv + (size_t)b * 512 : kbase + (size_t)(b - hq) * 256;
    const float* w1 = is_q ? q_w1 : k_w1;
    const float x = __half2float(src[d]);
    float ss = warp_sum(x * x);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += s_red[w];
    const float inv = rsqrtf(tot / 256.0f + eps);
    const float xn = round_f16(x * inv * w1[d]);
    s_n[d] = xn;
    __syncthreads();
    const float c = __half2float(cos_tab[(size_t)pos * 256 + d]);
    const float s = __half2float(sin_tab[(size_t)pos * 256 + d]);
    const float partner = (d < 128) ? -s_n[d + 128] : s_n[d - 128];
    const __half r = __float2half(round_f16(xn * c) + round_f16(partner * s));
    if (is_q) {
        q_out[(size_t)b * 256 + d] = r;
        gate_out[(size_t)b * 256 + d] = src[256 + d];
    } else {
        keys[((size_t)(b - hq) * max_len + pos) * 256 + d] = r;
    }
}

// Decode: the position is read from device memory.
__global__ void __launch_bounds__(256)
attn_prep_kernel(const __half* __restrict__ qkv, const float* __restrict__ q_w1,
                 const float* __restrict__ k_w1, const __half* __restrict__ cos_tab,
                 const __half* __restrict__ sin_tab, const long long* __restrict__ pos_ptr,
                 __half* __restrict__ q_out, __half* __restrict__ gate_out,
                 __half* __restrict__ keys, __half* __restrict__ values, int hq, int hkv,
                 int max_len, float eps) {
    pdl_prologue();
    PDL_FRESH(qkv); PDL_FRESH(q_w1); PDL_FRESH(k_w1); PDL_FRESH(cos_tab); PDL_FRESH(sin_tab); PDL_FRESH(pos_ptr);
    PDL_FRESH(q_out); PDL_FRESH(gate_out); PDL_FRESH(keys); PDL_FRESH(values);
    attn_prep_one_token(qkv, q_w1, k_w1, cos_tab, sin_tab, *pos_ptr, q_out, gate_out, keys, values,
                        hq, hkv, max_len, eps);
}

// Prefill: token blockIdx.y of a chunk starting at position pos0; qkv is token-major with `ld`
// halves between token rows, q_out / gate_out token-major [tokens][hq * 256].
__global__ void __launch_bounds__(256)
attn_prep_tokens_kernel(const __half* __restrict__ qkv, long long ld,
                        const float* __restrict__ q_w1, const float* __restrict__ k_w1,
                        const __half* __restrict__ cos_tab, const __half* __restrict__ sin_tab,
                        int pos0, __half* __restrict__ q_out, __half* __restrict__ gate_out,
                        __half* __restrict__ keys, __half* __restrict__ values, int hq, int hkv,
                        int max_len, float eps) {
    pdl_prologue();
    PDL_FRESH(qkv); PDL_FRESH(q_w1); PDL_FRESH(k_w1); PDL_FRESH(cos_tab); PDL_FRESH(sin_tab); PDL_FRESH(q_out);
    PDL_FRESH(gate_out); PDL_FRESH(keys); PDL_FRESH(values);
    const size_t t = blockIdx.y;
    attn_prep_one_token(qkv + t * (size_t)ld, q_w1, k_w1, cos_tab, sin_tab,
                        (long long)pos0 + (long long)t, q_out + t * (size_t)hq * 256,
                        gate_out + t * (size_t)hq * 256, keys, values, hq, hkv, max_len, eps);
}

// next = argmax(logits) (lowest index among equal maxima); also records the token and advances
// the position counters, so the next replay of the step graph needs no host input.
__global__ void __launch_bounds__(1024)
argmax_advance_kernel(const __half* __restrict__ logits, int vocab, long long* __restrict__ tok,
                      long long* __restrict__ pos, long long* __restrict__ len,
                      long long* __restrict__ history, long long* __restrict__ hist_count,
                      int hist_cap) {
    pdl_prologue();
    PDL_FRESH(logits); PDL_FRESH(tok); PDL_FRESH(pos); PDL_FRESH(len); PDL_FRESH(history); PDL_FRESH(hist_count);
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    // 8 logits per 16-byte load, 4 loads in flight per thread (logits is 16-byte aligned when it
    // is a whole allocation; otherwise the scalar loop below handles everything)
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        const int nvec = vocab >> 3;
        for (int v0 = t; v0 < nvec; v0 += 1024 * 4) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int vi = v0 + u * 1024;
                r[u] = (vi < nvec) ? *reinterpret_cast<const uint4*>(logits + (size_t)vi * 8)
                                   : make_uint4(0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int vi = v0 + u * 1024;
                const __half* h = reinterpret_cast<const __half*>(&r[u]);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const float v = __half2float(h[e]);
                    const int i = vi * 8 + e;
                    if (vi < nvec && (v > best || (v == best && i < bi))) { best = v; bi = i; }
                }
            }
        }
        done = nvec << 3;
    }
    for (int i = done + t; i < vocab; i += 1024) {
        const float v = __half2float(logits[i]);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { s_v[warp] = best; s_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = s_v[lane];
        bi = s_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            if (bi == 0x7fffffff) bi = 0;  // all-NaN logits
            *tok = bi;
            if (history && hist_count) {
                const long long n = *hist_count;
                if (n < hist_cap) history[n] = bi;
                *hist_count = n + 1;
            }
            if (pos) *pos += 1;
            if (len) *len += 1;
        }
    }
}

// h[i] = f16(f32(h[i]) + f32(y[i])): the residual add that follows the all-reduce of a K-split
// layer's partial outputs in tensor-parallel decode.
__global__ void __launch_bounds__(256)
residual_add_kernel(__half* __restrict__ h, const __half* __restrict__ y, int n) {
    pdl_prologue();
    PDL_FRESH(h); PDL_FRESH(y);
    const int i = (blockIdx.x * 256 + threadIdx.x) * 2;
    if (i + 1 < n) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(h + i));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(y + i));
        *reinterpret_cast<__half2*>(h + i) = __floats2half2_rn(a.x + b.x, a.y + b.y);
    } else if (i < n) {
        h[i] = __float2half(__half2float(h[i]) + __half2float(y[i]));
    }
}

// Tensor-parallel greedy pick: every rank has the (value, global index) of its vocabulary slice's
// maximum; cand holds all ranks' pairs [world][2] as fp32 (index stored exactly: vocab < 2^24).
__global__ void pick_global_argmax_kernel(const float* __restrict__ cand, int world,
                                          long long* __restrict__ tok, long long* __restrict__ pos,
                                          long long* __restrict__ len,
                                          long long* __restrict__ history,
                                          long long* __restrict__ hist_count, int hist_cap) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float best = -INFINITY;
    long long bi = 0;
    for (int r = 0; r < world; r++) {
        const float v = cand[2 * r];
        const long long i = (long long)cand[2 * r + 1];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    *tok = bi;
    if (history && hist_count) {
        const long long n = *hist_count;
        if (n < hist_cap) history[n] = bi;
        *hist_count = n + 1;
    }
    if (pos) *pos += 1;
    if (len) *len += 1;
}

// local argmax of a vocabulary slice -> cand[0] = value, cand[1] = offset + index
__global__ void __launch_bounds__(1024)
argmax_slice_kernel(const __half* __restrict__ logits, int vocab, long long offset,
                    float* __restrict__ cand) {
    pdl_prologue();
    PDL_FRESH(logits); PDL_FRESH(cand);
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = t; i < vocab; i += 1024) {
        const float v = __half2float(logits[i]);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { s_v[warp] = best; s_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = s_v[lane];
        bi = s_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            if (bi == 0x7fffffff) bi = 0;
            cand[0] = best;
            cand[1] = (float)(offset + bi);
        }
    }
}

}  // namespace nvfp4

extern "C" {

// h, y fp16 [n]: h += y (fp32 add, one rounding).  0 / -1.
int launch_residual_add(void* h, const void* y, int n, void* stream) {
    if (!h || !y || n <= 0) return -1;
    return nvfp4::launch_pdl(nvfp4::residual_add_kernel, dim3((n + 511) / 512), dim3(256), 0,
                             (cudaStream_t)stream, (__half*)h, (const __half*)y, n) == cudaSuccess
               ? 0 : -1;
}

// Tensor-parallel argmax, step 1: cand (fp32 [2]) = (max of logits[0..vocab), offset + argmax).
int launch_argmax_slice(const void* logits, int vocab, long long offset, void* cand, void* stream) {
    if (!logits || !cand || vocab <= 0 || offset < 0 || offset + vocab > (1 << 24)) return -1;
    nvfp4::argmax_slice_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>((const __half*)logits, vocab,
                                                                     offset, (float*)cand);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Step 2, after an all-gather of every rank's cand pair into cand_all (fp32 [world, 2]): pick the
// global maximum (lowest index among equals) and advance the step counters as
// launch_argmax_advance does.
int launch_pick_global_argmax(const void* cand_all, int world, void* tok, void* pos, void* len,
                              void* history, void* hist_count, int hist_cap, void* stream) {
    if (!cand_all || !tok || world <= 0) return -1;
    nvfp4::pick_global_argmax_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(
        (const float*)cand_all, world, (long long*)tok, (long long*)pos, (long long*)len,
        (long long*)history, (long long*)hist_count, hist_cap);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// table fp16 [vocab, hidden]; tok: device int64; out fp16 [hidden].  0, or -1 bad args / launch.
int launch_embed_gather(const void* table, const void* tok, void* out, int hidden, long long vocab,
                        void* stream) {
    if (!table || !tok || !out || hidden <= 0 || vocab <= 0) return -1;
    const int per = 256 * 8;
    return nvfp4::launch_pdl(nvfp4::embed_gather_kernel, dim3((hidden + per - 1) / per), dim3(256), 0,
                             (cudaStream_t)stream, (const __half*)table, (const long long*)tok,
                             (__half*)out, hidden, vocab) == cudaSuccess ? 0 : -1;
}

// qkv fp16 [hq*512 + 2*hkv*256]; q_w1, k_w1 fp32 [256] (1 + weight); cos/sin tables fp16
// [max_len, 256]; pos: device int64 index of the current token; q_out, gate_out fp16 [hq*256];
// keys, values fp16 [hkv, max_len, 256].  0, or -1 bad args / launch error.
int launch_attn_prep(const void* qkv, const void* q_w1, const void* k_w1, const void* cos_tab,
                     const void* sin_tab, const void* pos, void* q_out, void* gate_out, void* keys,
                     void* values, int hq, int hkv, int max_len, float eps, void* stream) {
    if (!qkv || !q_w1 || !k_w1 || !cos_tab || !sin_tab || !pos || !q_out || !gate_out || !keys ||
        !values || hq <= 0 || hkv <= 0 || max_len <= 0)
        return -1;
    return nvfp4::launch_pdl(nvfp4::attn_prep_kernel, dim3(hq + 2 * hkv), dim3(256), 0,
                             (cudaStream_t)stream, (const __half*)qkv, (const float*)q_w1,
                             (const float*)k_w1, (const __half*)cos_tab, (const __half*)sin_tab,
                             (const long long*)pos, (__half*)q_out, (__half*)gate_out, (__half*)keys,
                             (__half*)values, hq, hkv, max_len, eps) == cudaSuccess ? 0 : -1;
}

// The same for the n_tokens tokens of a prefill chunk that starts at position pos0 (host value):
// qkv token-major with `ld` halves between rows; q_out, gate_out token-major [n_tokens][hq*256];
// token i writes cache row pos0 + i.  0, or -1 bad args / launch error.
int launch_attn_prep_tokens(const void* qkv, long long ld, const void* q_w1, const void* k_w1,
                            const void* cos_tab, const void* sin_tab, int pos0, int n_tokens,
                            void* q_out, void* gate_out, void* keys, void* values, int hq, int hkv,
                            int max_len, float eps, void* stream) {
    if (!qkv || !q_w1 || !k_w1 || !cos_tab || !sin_tab || !q_out || !gate_out || !keys || !values ||
        hq <= 0 || hkv <= 0 || max_len <= 0 || n_tokens <= 0 || n_tokens > 65535 || pos0 < 0 ||
        pos0 + n_tokens > max_len || ld < (long long)hq * 512 + 2LL * hkv * 256)
        return -1;
    return nvfp4::launch_pdl(nvfp4::attn_prep_tokens_kernel, dim3(hq + 2 * hkv, n_tokens),
                             dim3(256), 0, (cudaStream_t)stream, (const __half*)qkv, ld,
                             (const float*)q_w1, (const float*)k_w1, (const __half*)cos_tab,
                             (const __half*)sin_tab, pos0, (__half*)q_out, (__half*)gate_out,
                             (__half*)keys, (__half*)values, hq, hkv, max_len, eps) == cudaSuccess
               ? 0 : -1;
}

// logits fp16 [vocab]; tok/pos/len/hist_count: device int64 scalars (pos, len, history and
// hist_count may be NULL); history: device int64 [hist_cap].  0, or -1.
int launch_argmax_advance(const void* logits, int vocab, void* tok, void* pos, void* len,
                          void* history, void* hist_count, int hist_cap, void* stream) {
    if (!logits || !tok || vocab <= 0) return -1;
    return nvfp4::launch_pdl(nvfp4::argmax_advance_kernel, dim3(1), dim3(1024), 0,
                             (cudaStream_t)stream, (const __half*)logits, vocab, (long long*)tok,
                             (long long*)pos, (long long*)len, (long long*)history,
                             (long long*)hist_count, hist_cap) == cudaSuccess ? 0 : -1;
}

}  // extern "C"

/* C ABI of libnvfp4_b200.so — the sm_100a replacement for the reference's six ctypes DLLs.
 *
 * Every function is `extern "C"`, takes plain pointers and sizes, and (unless stated otherwise)
 * only enqueues work on the stream it is given: no allocation, no synchronisation, safe to call
 * while that stream is being captured into a CUDA graph.  Device pointers are raw addresses
 * (ctypes c_void_p built from tensor.data_ptr()); `stream` is a cudaStream_t passed as void*.
 *
 * Citations give the reference interface each entry point replaces (path within the reference
 * project : line).
 */
#ifndef NVFP4_B200_H
#define NVFP4_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------------------------------
 * Device memory helpers.  kernels/nvfp4_gemv.cu:820-835, kernels/nvfp4_cuda_v5.cu:424-457.
 * gpu_malloc returns NULL on failure.  The copies are synchronous and return the cudaError_t as
 * an int (0 = success).  The caller owns the memory and may do byte arithmetic on the address.
 * ------------------------------------------------------------------------------------------- */
void* gpu_malloc(size_t bytes);
void gpu_free(void* p);
int gpu_memcpy_h2d(void* dst, const void* src, size_t bytes);
int gpu_memcpy_d2h(void* dst, const void* src, size_t bytes);
int gpu_memcpy_d2d(void* dst, const void* src, size_t bytes);  /* no counterpart in the reference */
int gpu_sync(void);                                              /* kernels/nvfp4_cuda_v5.cu:433 */
int get_gpu_info(char* name_buf, int buf_size, int* cc_major, int* cc_minor); /* :447-457 */
int nvfp4_b200_abi_version(void);                    /* no counterpart in the reference */

/* ---------------------------------------------------------------------------------------------
 * Batch-1 GEMV: output[M] (fp16) = W[M,K] . activation[K] (fp16), fp32 accumulation.
 *   weight_packed [M, K/2] u8 (element 2i = low nibble of byte i), weight_scales [M, K/16] u8.
 * Returns 0; -2 if K % 32 != 0, M <= 0, a pointer is NULL, weight_packed/activation are not
 * 16-byte aligned or weight_scales is not 2-byte aligned; -1 if the launch failed.
 * All generations of the reference kernel share one implementation here.
 * kernels/nvfp4_gemv.cu:837-851 (v1), :929-943 (v8), :946-961 (v4), :854-877 (v5), :880-895 (v6),
 * :898-926 (v7, additionally K % 64 == 0), :964-977 (nl).
 * ------------------------------------------------------------------------------------------- */
int launch_nvfp4_gemv(const void* weight_packed, const void* weight_scales, const void* activation,
                      void* output, int M, int K, void* stream);
int launch_nvfp4_gemv_v8(const void* weight_packed, const void* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream);
int launch_nvfp4_gemv_v4(const void* weight_packed, const void* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream);
int launch_nvfp4_gemv_v5(const void* weight_packed, const void* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream);
int launch_nvfp4_gemv_v6(const void* weight_packed, const void* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream);
int launch_nvfp4_gemv_v7(const void* weight_packed, const void* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream);
int launch_nvfp4_gemvnl(const void* weight_packed, const void* weight_scales,
                        const void* activation, void* output, int M, int K, void* stream);

/* Two activations, one pass over the weights: output[2, M], output[m] = W[m,:].act0,
 * output[M + m] = W[m,:].act1.  kernels/nvfp4_gemv.cu:979-994. */
int launch_nvfp4_gemv2(const void* weight_packed, const void* weight_scales, const void* act0,
                       const void* act1, void* output, int M, int K, void* stream);

/* The same with the two activations interleaved as K fp16 pairs (act_i[2k] = act0[k],
 * act_i[2k + 1] = act1[k]); output[2, M].  kernels/nvfp4_gemv.cu:997-1011. */
int launch_nvfp4_gemv2i(const void* weight_packed, const void* weight_scales, const void* act_i,
                        void* output, int M, int K, void* stream);

/* Dense GEMM for more than two tokens: output[M, N] (fp16) = dequant(W)[M, K] . activation[K, N]
 * (fp16, N = tokens, token-minor as the reference's caller prepares it).  Weight x block scale in
 * fp16, fp16 x fp16 products, fp32 accumulation, as the reference's wmma kernel.  Runs on tcgen05
 * tensor cores when K % 64 == 0, N % 8 == 0 and the pointers are 16-byte aligned (scales 4-byte),
 * otherwise on a CUDA-core kernel.  Returns 0 or the cudaError_t of the launch; -2 for K % 16 != 0,
 * non-positive sizes or NULL pointers.  kernels/nvfp4_cuda_v5.cu:406-422. */
int launch_nvfp4_gemmtc_v5(const uint8_t* d_weight_packed, const uint8_t* d_weight_scales,
                           const void* d_activation, void* d_output, int M, int N, int K,
                           void* stream);
/* The same product for a caller that keeps tokens as rows (the chunked prefill; the reference's
 * caller transposes through torch around launch_nvfp4_gemmtc_v5, pipeline/_qwen38_infer.py:175-181).
 * flags bit 0: act is token-major act[n_tokens][ld_act] (else act[K][ld_act], tokens minor);
 * bit 1: out is token-major out[n_tokens][ld_out] (else out[M][ld_out]); bit 2 (needs bit 1):
 * out[t][m] += result, the decoder layer's residual add (the fp16-rounded result added in fp32 and
 * rounded once more: exactly what a separate add of the fp16 GEMM output gives).  Same arithmetic
 * and accumulation order as launch_nvfp4_gemmtc_v5: the outputs are bit-identical to transposing
 * around it.  Tensor-core kernel only: K % 64 == 0, ld_act % 8 == 0, 16-byte aligned act and
 * weights, a feature-major side has ld == n_tokens rounded up to 8 (its columns past n_tokens are
 * read as / written with zeros).  0; -2 for anything else; -3 no tensor-map encoder; or the
 * launch's cudaError_t. */
int launch_nvfp4_gemm_w4a16_ex(const uint8_t* d_weight_packed, const uint8_t* d_weight_scales,
                               const void* act, long long ld_act, void* out, long long ld_out, int M,
                               int n_tokens, int K, int flags, void* stream);
int get_kernel_shared_mem_bytes(void);                          /* kernels/nvfp4_cuda_v5.cu:460-464 */
/* 0 if no bounded wait inside the tensor-core GEMM ever ran out; 1 + wait id otherwise.  reset != 0
 * clears it.  Synchronous.  No counterpart in the reference. */
int nvfp4_gemm_status(int reset);
/* Tuning hook of the W4A16 GEMM entry points.  Bit 0: 256-row CTA tiles (two accumulators in tensor
 * memory, the activation tile fetched once for twice the rows) for more than 128 tokens when they
 * still give every SM a CTA.  Bit 1: the CTA-pair kernel (clusters of two CTAs, tcgen05
 * cta_group::2: each CTA dequantises 128 rows and loads half of a 256-token tile) for shapes of more
 * than 128 tokens that do not get 256-row tiles.  Bit 2: the CTA-pair kernel wherever it can run
 * (more than 128 tokens, K % 128 == 0).  Default 3.  All kernels give bit-identical results. */
void nvfp4_b200_gemm_config(int flags);

/* Tuning hook; no counterpart in the reference.  warps per CTA (0 = auto, 2, 4 or 8), resident
 * CTAs per SM used to size the grid (0 = planner; above 64 = an exact grid size), flags: bit 0 routes every GEMV to
 * the non-tensor-core kernel, bit 1 turns programmatic dependent launch off, bits 4..6 cap and
 * bits 8..10 force the cluster K split (1, 2 or 4 CTAs per row tile; 0 = planner decides).
 * Process-wide, not thread-safe.  Returns 0 or -2. */
int nvfp4_b200_gemv_config(int warps, int ctas_per_sm, int flags);

/* Two kernels serve the batch-1 GEMV.  The default streams the weights through registers
 * (gemv_mma_kernel).  The second streams them through per-warp shared-memory rings filled by TMA
 * tensor copies (gemv_stream_kernel; K % 256 == 0, weight_scales 16-byte aligned); it is off by
 * default because it measured slower on B200 at every 27B layer shape, and is kept for its
 * attribution probes and as the base of a persistent variant.  Neither function below has a
 * counterpart in the reference.
 * nvfp4_gemv_status: 0 if no bounded wait inside the ring kernel ever ran out; 1 + wait id
 * otherwise (1 a warp waiting for a stage's bytes, 3 final drain, 4 a tile's partial-sum slot still
 * in use).  reset != 0 clears it.  Synchronous.
 * nvfp4_b200_gemv_stream_config: flags bit 0 turns the ring kernel on for the shapes it takes;
 * bits 4 and 5 are attribution probes that give WRONG results on purpose (bit 4: no arithmetic, a
 * launch costs what its weight stream costs; bit 5: no weight copies, a launch costs what its
 * arithmetic costs), the counterpart of the compile-time probes in kernels/nvfp4_gemv.cu:25-33.
 * warps per CTA (0 = 8; 4, 8, 12), shared-memory budget per CTA in KB (0 = 208 with one CTA per SM,
 * 98 with two), stage size in KB (0 = 9), most stages per warp (0 = 4; 2..4), CTAs per SM that size
 * the grid (0 = 1; 1, 2), unit in which rows are dealt to the CTAs (0 = 4; 4, 16).  Process-wide,
 * not thread-safe.  Returns 0 or -2.
 *
 * Contract of every GEMV launcher under programmatic dependent launch (on by default): weights,
 * scales and norm weights may be read BEFORE the previous kernel in the stream has finished, so
 * they must not be written by a kernel launched earlier in the same stream without a full
 * dependency in between (an event, a synchronisation, or a launch with bit 1 of
 * nvfp4_b200_gemv_config's flags set).  Activations, residuals and outputs are only touched after
 * the previous kernel has completed. */
int nvfp4_gemv_status(int reset);
int nvfp4_b200_gemv_stream_config(int warps, int smem_kb, int stage_kb, int min_stages,
                                  int ctas_per_sm, int rows_per_box, int flags);

/* ---------------------------------------------------------------------------------------------
 * Zero-centred RMSNorm: out[r, :] = f16( f32(x[r, :]) * rsqrt(mean(x^2) + eps) * w1 ).
 * x fp16, row r starts at x + r*row_stride (elements); w1 fp32 [n] = 1 + weight; out fp16
 * contiguous [rows, n].  Returns -1 for rows <= 0, n <= 0 or a NULL pointer, else the cudaError_t.
 * kernels/nvfp4_rmsnorm.cu:65-76.
 * ------------------------------------------------------------------------------------------- */
int launch_rmsnorm(const void* x, long long row_stride, const void* w1, void* out, int rows, int n,
                   float eps, void* stream);

/* RoPE (full rotation over 256 dims) on q [hq, 256] and k [hkv, 256] fp16 with cos/sin fp16 [256]:
 * out = f16(f16(v*cos) + f16(rotate_half(v)*sin)).  0; -1 bad arguments; -2 launch error.
 * kernels/nvfp4_rope_silu.cu:70-81. */
int launch_rope_qk(const void* q, const void* k, const void* cos, const void* sin, void* q_out,
                   void* k_out, int hq, int hkv, void* stream);

/* out[i] = f16( f32(f16(g/(1+exp(-g)))) * u ), g/u/out fp16 [n].  0; -1; -2 as above.
 * kernels/nvfp4_rope_silu.cu:83-91. */
int launch_silu_mul(const void* g, const void* u, void* out, int n, void* stream);

/* GQA attention decode (24 query heads, 4 KV heads, head dim 256) over a static KV cache, with the
 * sigmoid output gate.  q/gate/out fp16 [24*256]; keys/values fp16 [4, max_len, 256]; cum_len is a
 * DEVICE int64 holding the number of valid keys including the current token (read at run time, so
 * a captured graph follows the growing cache).  max_len is a run-time value here (the reference
 * compiles one DLL per length); -2 if max_len <= 0, max_len > 47104 or a pointer is NULL; else the
 * cudaError_t.  kernels/nvfp4_attn_decode.cu:121-132. */
int launch_attn_decode(const void* q, const void* keys, const void* values, const void* cum_len,
                       const void* gate, void* out, int max_len, float scale, void* stream);

/* launch_attn_decode for hq query heads and hkv KV heads (hq a multiple of hkv, head dim 256): a
 * tensor-parallel shard or a smaller model.  No counterpart in the reference (single GPU, fixed
 * 24/4 heads); the kernel is launch_attn_decode's.  -2 also for invalid head counts. */
int launch_attn_decode_heads(const void* q, const void* keys, const void* values,
                             const void* cum_len, const void* gate, void* out, int max_len, int hq,
                             int hkv, float scale, void* stream);

/* One Gated-DeltaNet decode step (16 key heads, 48 value heads, dim 128, conv kernel 4).
 * mixed fp16 [10240] = [q 2048 | k 2048 | v 6144]; z fp16 [6144]; b, a fp16 [48];
 * conv_w fp16 [10240*4]; conv_state fp16 [10240*4] in/out (layout c*4 + t);
 * A_log, dt_bias fp16 [48]; norm_w fp16 [128]; state fp32 [48*128*128] in/out, transposed
 * (value-dim major); scratch fp32 [10240] caller-provided workspace; out fp16 [6144].
 * Returns 0, or -1 on a NULL pointer or launch error.  kernels/nvfp4_dn_fused.cu:156-176. */
int launch_dn_fused(const void* mixed, const void* z, const void* b, const void* a,
                    const void* conv_w, void* conv_state, const void* A_log, const void* dt_bias,
                    const void* norm_w, void* state, void* scratch, void* out, float rms_eps,
                    void* stream);

/* The same step on a tensor-parallel shard holding n_kheads key heads and n_vheads value heads
 * (n_vheads a multiple of n_kheads; the full model is 16 / 48): mixed is
 * [q n_k*128 | k n_k*128 | v n_v*128], scratch holds (2 n_k + n_v)*128 floats, the other buffers
 * shrink the same way.  -1 also for invalid head counts.  No counterpart in the reference (it
 * has no multi-GPU path); the arithmetic is launch_dn_fused's. */
int launch_dn_fused_heads(const void* mixed, const void* z, const void* b, const void* a,
                          const void* conv_w, void* conv_state, const void* A_log,
                          const void* dt_bias, const void* norm_w, void* state, void* scratch,
                          void* out, int n_kheads, int n_vheads, float rms_eps, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Decode-engine entry points.  None has a C counterpart in the reference: there the same work is
 * done by PyTorch operators inside the captured model forward (pipeline/_qwen38_infer.py:679-685)
 * and by the monkey-patched module forwards (:456-479, :612-644, experiments/_qwen38_p9_fuse.py).
 * They exist so that a whole decode step is a fixed list of launches with no host work between.
 * ------------------------------------------------------------------------------------------- */

/* GEMV with fused neighbours.  prologue 1: the activation is first RMS-normalised with norm_w1
 * (fp32 [K], 1 + weight) and eps, arithmetic of launch_rmsnorm.  epilogue 1: output =
 * f16(residual + f16(y)), residual fp16 [M].  epilogue 2: weight rows are gate and up rows
 * interleaved in groups of 8 (rows 16j..16j+7 = gate rows 8j..8j+7, rows 16j+8..16j+15 = up rows
 * 8j..8j+7, M = 2 * outputs, M % 16 == 0) and output[8j+r] = silu(gate)*up with the arithmetic of
 * launch_silu_mul.  Requires K % 128 == 0, weights 32-byte, scales 8-byte, activation 16-byte
 * aligned; with prologue 1 also K <= 10240.  0; -2 bad arguments; -1 launch error. */
int launch_nvfp4_gemv_fused(const void* weight_packed, const void* weight_scales,
                            const void* activation, void* output, int M, int K, int prologue,
                            const void* norm_w1, float eps, int epilogue, const void* residual,
                            void* stream);

/* launch_attn_decode_heads with the keys of every head split over eight CTAs (no counterpart in
 * the reference): each warp requests its key AND value rows at once, partial softmax results are
 * combined in shared memory, then by the last CTA of a head to finish (in split order, so the
 * result does not depend on arrival order).  scratch: nvfp4_attn_split_scratch_bytes(hq) bytes,
 * 16-byte aligned, zeroed once before first use; calls sharing it must not overlap.  Results
 * match launch_attn_decode_heads to the last fp32 bit before the fp16 rounding.
 * 0; -2 bad arguments; else the launch error. */
long long nvfp4_attn_split_scratch_bytes(int hq);
int launch_attn_decode_split(const void* q, const void* keys, const void* values,
                             const void* cum_len, const void* gate, void* out, void* scratch,
                             int max_len, int hq, int hkv, float scale, void* stream);

/* out[hidden] = table[*tok] — table fp16 [vocab, hidden], tok a device int64.  0 / -1. */
int launch_embed_gather(const void* table, const void* tok, void* out, int hidden, long long vocab,
                        void* stream);

/* Between the q/k/v projection and launch_attn_decode: per-head RMSNorm of q and k (q_w1, k_w1
 * fp32 [256]), RoPE at position *pos from cos/sin tables fp16 [max_len, 256], k and v written into
 * the cache at *pos, the per-head gate halves of the q projection gathered into gate_out.
 * qkv fp16 [hq*512 + 2*hkv*256] = [per head q256|gate256][k][v]; pos a device int64.  0 / -1. */
int launch_attn_prep(const void* qkv, const void* q_w1, const void* k_w1, const void* cos_tab,
                     const void* sin_tab, const void* pos, void* q_out, void* gate_out, void* keys,
                     void* values, int hq, int hkv, int max_len, float eps, void* stream);

/* *tok = argmax(logits fp16 [vocab]) (lowest index among equal maxima); appends it to history
 * (device int64 [hist_cap], counter hist_count) and increments *pos and *len (device int64; any
 * of pos, len, history, hist_count may be NULL).  0 / -1. */
int launch_argmax_advance(const void* logits, int vocab, void* tok, void* pos, void* len,
                          void* history, void* hist_count, int hist_cap, void* stream);

/* Tensor-parallel glue (the reference has no multi-GPU path): h += y after the all-reduce of a
 * K-split layer (fp16 [n], fp32 add, one rounding); per-rank argmax of a vocabulary slice into an
 * fp32 pair (value, offset + index; offset + vocab <= 2^24); and the pick of the global maximum from
 * all ranks' pairs (fp32 [world, 2]) with the counter updates of launch_argmax_advance.  0 / -1. */
int launch_residual_add(void* h, const void* y, int n, void* stream);
int launch_argmax_slice(const void* logits, int vocab, long long offset, void* cand, void* stream);
int launch_pick_global_argmax(const void* cand_all, int world, void* tok, void* pos, void* len,
                              void* history, void* hist_count, int hist_cap, void* stream);

/* One-shot all-reduce + residual add over NVLink peer memory (no counterpart in the reference).
 * Each rank owns a communication buffer (gpu_malloc of nvfp4_comm_buffer_bytes(n), zeroed by
 * nvfp4_comm_init) that the other ranks map through CUDA IPC (nvfp4_ipc_get_handle gives the
 * 64-byte handle, nvfp4_ipc_open_handle maps a peer's).  The K-split GEMV writes its partial
 * vector into its own buffer at nvfp4_comm_data_offset(n, parity); launch_allreduce_residual then
 * signals the peers, waits for them with a bounded spin, pulls their vectors with peer loads and
 * does h += f16(sum over ranks, fp32, rank order).  parity alternates 0, 1, 0, ... over the calls;
 * every rank makes the same sequence of calls.  bufs is a HOST array of `world` device pointers
 * (rank r's buffer as mapped in this process).  world <= 8, n % 8 == 0.  nvfp4_comm_status returns
 * 0, or 1 + r if peer r failed to arrive within the spin limit at some call.
 * launch_nvfp4_gemv_allreduce fuses the K-split GEMV itself with that all-reduce: h[M] +=
 * f16(sum over ranks of W_r . act_r) in ONE kernel — each CTA stores its tile's partial outputs
 * into every rank's buffer (peer stores, overlapping the remaining tiles), the last CTA to finish
 * exchanges flags with the peers (bounded wait; status 101 + r on timeout) and applies the sum to
 * h.  M % 16 == 0, M <= n, K % 128 == 0, GEMV alignment rules; -2 bad arguments, -1 launch error. */
int launch_nvfp4_gemv_allreduce(const void* weight_packed, const void* weight_scales,
                                const void* activation, void* h, int M, int K,
                                const void* const* bufs, int rank, int world, int n, int parity,
                                void* stream);
/* The all-reduce inside the CONSUMING GEMV: h (fp16 [K], in/out) first receives the sum over the
 * ranks of the partial vectors in data slot `parity` (CTA 0 exchanges flags with the peers and
 * pulls their vectors over NVLink while every CTA's first weight loads are in flight; the other
 * CTAs wait, bounded, for CTA 0's sequence number), then is RMS-normalised with norm_w1 and
 * multiplied: one launch per K-split layer less than launch_allreduce_residual + fused GEMV.
 * epilogue 0 or 2 as in launch_nvfp4_gemv_fused.  epoch: device u32 counting decode steps; site,
 * n_sites: this call's place among a step's all-reduces (same on every rank).  K <= n, K <= 10240.
 * launch_argmax_exchange: greedy pick over the ranks' vocabulary slices in one launch (local
 * argmax, pairs pushed to every peer, bounded wait, global pick, history and counters advanced,
 * *epoch += 1); logits fp16 [vocab] is this rank's slice starting at global index offset.
 * Status codes in nvfp4_comm_status: 201 + r / 301 + r peer r missing, 299 CTA 0 never published. */
int launch_nvfp4_gemv_fused_ar(const void* weight_packed, const void* weight_scales, void* h,
                               void* output, int M, int K, const void* norm_w1, float eps,
                               int epilogue, const void* const* bufs, int rank, int world, int n,
                               int parity, const void* epoch, int site, int n_sites, void* stream);
int launch_argmax_exchange(const void* logits, int vocab, long long offset,
                           const void* const* bufs, int rank, int world, int n, void* epoch,
                           void* tok, void* pos, void* len, void* history, void* hist_count,
                           int hist_cap, void* stream);
long long nvfp4_comm_buffer_bytes(int n);
long long nvfp4_comm_data_offset(int n, int parity);
int nvfp4_comm_init(void* buf, int n);
int nvfp4_ipc_get_handle(void* dev_ptr, void* handle_out);
void* nvfp4_ipc_open_handle(const void* handle);
int nvfp4_ipc_close_handle(void* p);
int nvfp4_comm_status(const void* my_buf);
int launch_allreduce_residual(void* h, const void* const* bufs, int rank, int world, int n,
                              int parity, void* stream);

/* Chunked prefill (no counterpart in the reference, which prefills through the third-party model
 * code with launch_nvfp4_gemmtc_v5 as its Linear: pipeline/_qwen38_infer.py:796-809).  A chunk's
 * activations are token-major [tokens][features] between operators and token-minor
 * [features][tokens] at the GEMM; every operator keeps the arithmetic of its decode-step twin.
 *   launch_transpose_f16   dst[c][r] = src[r][c] (r < R, c < C); dst rows ld_dst >= R long, tail zeroed
 *   launch_add_transposed  h[t][c] += dT[c][t] (fp32 add, one rounding): residual add from a GEMM output
 *   launch_embed_rows      out[t][:] = table[ids[t]], ids device int64 [n]
 *   launch_silu_mul_rows   gu token-minor [2*inter][N], gate/up rows interleaved by 8 -> act [inter][N]
 *   launch_attn_prep_tokens  launch_attn_prep for the n_tokens rows of a chunk starting at position
 *                          pos0 (host int); qkv token-major, ld halves per row; q_out/gate_out
 *                          token-major [n_tokens][hq*256]; token i writes cache row pos0 + i
 *   launch_attn_prefill    causal attention, decode arithmetic: token i attends to cache rows
 *                          [0, len0 + i); q, gate, out token-major [n_tokens][hq*256]
 *   launch_dn_prefill      one Gated-DeltaNet layer over n tokens: x token-major [n][ld], row =
 *                          [mixed | z | b | a]; conv window and recurrent state carried in
 *                          conv_state / state; out token-major [n][nv*128]; work: 256-byte aligned
 *                          scratch of nvfp4_dn_prefill_work_bytes(n, nk, nv) bytes
 * All return 0, -1 for bad arguments (launch_attn_prefill: -2), or a launch error code. */
int launch_transpose_f16(const void* src, long long ld_src, void* dst, long long ld_dst, int R,
                         int C, void* stream);
int launch_add_transposed(void* h, const void* dT, long long ldT, int n, int C, void* stream);
int launch_embed_rows(const void* table, const void* ids, void* out, int n, int hidden,
                      long long vocab, void* stream);
int launch_silu_mul_rows(const void* gu, void* act, int inter, int N, void* stream);
int launch_attn_prep_tokens(const void* qkv, long long ld, const void* q_w1, const void* k_w1,
                            const void* cos_tab, const void* sin_tab, int pos0, int n_tokens,
                            void* q_out, void* gate_out, void* keys, void* values, int hq, int hkv,
                            int max_len, float eps, void* stream);
int launch_attn_prefill(const void* q, const void* keys, const void* values, int len0,
                        int n_tokens, const void* gate, void* out, int max_len, int hq, int hkv,
                        float scale, void* stream);
long long nvfp4_dn_prefill_work_bytes(int n, int nk, int nv);
int launch_dn_prefill(const void* x, long long ld, const void* conv_w, void* conv_state,
                      const void* A_log, const void* dt_bias, const void* norm_w, void* state,
                      void* work, long long work_bytes, void* out, int n, int nk, int nv,
                      float rms_eps, void* stream);

/* Quantiser on the device: src fp16 [M, K] row-major -> packed [M, K/2] + scales [M, K/16], byte
 * for byte what the reference's CPU codec produces (scale exponent ceil(log2(max/6)), zero block
 * -> byte 127, nearest code with ties to the smaller code, -0 -> +0): codec/nvfp4_codec.py:166-245,
 * codec/nvfp4_codec_fast.py:19-53, pipeline/_qwen38_nvfp4_pack.py:34-67.  The reference has no GPU
 * entry for this; it makes container production and activation quantisation a stream-speed step.
 * K % 16 == 0, src 16-byte aligned, packed 8-byte aligned.  Asynchronous, capturable.
 * 0; -2 bad shape or pointer; -1 launch error. */
int launch_nvfp4_encode(const void* src_fp16, void* packed, void* scales, int M, int K,
                        void* stream);

/* Dequantiser on the device: out[r][0..K) fp16 = row ids[r] of an NVFP4 table (packed
 * [table_rows][K/2], scales [table_rows][K/16]); ids a device int64 array, or NULL for rows
 * 0..n_rows-1.  Bit for bit the reference's CPU decoder (code point x 2^(byte-127) in float64, one
 * rounding to fp16): codec/nvfp4_codec.py:248-275, pipeline/_qwen38_infer.py:117-128 (the packed
 * embedding table, which the reference decodes on the host per token).  K % 16 == 0; packed 8-byte,
 * out 16-byte aligned.  0; -2 bad arguments; -1 launch error. */
int launch_nvfp4_decode_rows(const void* packed, const void* scales, const void* ids, void* out,
                             int n_rows, int K, long long table_rows, void* stream);

/* GEMV on the FP4 tensor-core path: output[M] (fp16) = dequant(W)[M, K] . activation[K] (fp16), the
 * semantics of launch_nvfp4_gemv_v8 (kernels/nvfp4_gemv.cu:88-100).  Weight and scale bytes go
 * HBM -> shared memory (TMA) -> tcgen05.mma kind::mxf4nvf4 without passing through registers; the
 * fp16 activation enters as 16 exact base-4 digit columns, so the products are those of the W4A16
 * rule with fp32 accumulation.  K % 256 == 0; weight pointers and activation 16-byte aligned.  The
 * first call on a device allocates a workspace (do it outside stream capture).  0; -2 shape or
 * pointer not taken; -3 no tensor-map encoder / no memory; else the launch's cudaError_t.
 * nvfp4_gemv_tc_status: 0, or 1 + id of the first bounded wait in that kernel that ran out. */
int launch_nvfp4_gemv_tc(const uint8_t* weight_packed, const uint8_t* weight_scales,
                         const void* activation, void* output, int M, int K, void* stream);
/* The same with the neighbours of launch_nvfp4_gemv_fused: prologue 1 = RMSNorm of the activation
 * (norm_w1 fp32 [K], 16-byte aligned, K <= 11520), epilogue 1 = residual add, epilogue 2 =
 * silu(gate) * up over interleaved gate / up rows (M % 16 == 0).  Same return values. */
int launch_nvfp4_gemv_tc_fused(const uint8_t* weight_packed, const uint8_t* weight_scales,
                               const void* activation, void* output, int M, int K, int prologue,
                               const void* norm_w1, float eps, int epilogue, const void* residual,
                               void* stream);
/* The MLP block of a decoder layer in ONE launch of the tensor-core GEMV kernel: act[inter] =
 * silu(gate) * up over W_gu . rmsnorm(h) (W_gu = [2 inter][hidden], gate / up rows interleaved in
 * groups of 8, norm_w1 fp32 [hidden] = 1 + weight), then h[hidden] += W_down . act (W_down =
 * [hidden][inter]); the weight ring streams on from the first matrix into the second across a
 * bounded grid-wide barrier.  Results are those of launch_nvfp4_gemv_tc_fused(prologue 1, epilogue
 * 2) followed by (prologue 0, epilogue 1).  hidden, inter % 256 == 0, hidden <= 11520, all pointers
 * 16-byte aligned.  Return values of launch_nvfp4_gemv_tc. */
int launch_nvfp4_mlp_tc(const uint8_t* gu_packed, const uint8_t* gu_scales, const uint8_t* down_packed,
                        const uint8_t* down_scales, void* h, void* act, const void* norm_w1, float eps,
                        int inter, int hidden, void* stream);
int nvfp4_gemv_tc_status(int reset);
/* Routing: launch_nvfp4_gemv_fused hands calls with M * K >= min_mega_elements * 2^20 to the
 * tensor-core kernel when shape and alignment allow (nvfp4_b200_gemv_tc_config; 0 = never; default
 * 35), launch_nvfp4_gemv_v8 those above its own threshold (nvfp4_b200_gemv_tc_config_plain; default
 * 40: timed back to back on cold activations the register-streaming kernel wins below that).  nvfp4_gemv_tc_wanted / _plain: the rules, 1 or 0.  nvfp4_gemv_tc_prepare: allocate the
 * current device's workspace now, outside any stream capture (0 or -3). */
void nvfp4_b200_gemv_tc_config(int min_mega_elements);
/* Weight-ring depth of the tensor-core GEMV: 5 stages (default) or 3. */
void nvfp4_b200_gemv_tc_ring(int stages);
/* Weight stages a CTA of the tensor-core GEMV requests at kernel entry (1..5, default 2); the rest
 * follow its activation loads. */
void nvfp4_b200_gemv_tc_prefetch(int stages_at_entry);
/* CTAs of one tensor-core GEMV launch per SM: 2 (default) or 1. */
void nvfp4_b200_gemv_tc_ctas(int per_sm);
int nvfp4_gemv_tc_wanted(int M, int K);
int nvfp4_gemv_tc_wanted_plain(int M, int K);
void nvfp4_b200_gemv_tc_config_plain(int min_mega_elements);
int nvfp4_gemv_tc_prepare(void);
/* Timing probe of launch_nvfp4_gemv_tc: while a device buffer of 128 int64 words is set, launch n
 * folds into words 16 (n % 8) .. the global nanosecond timer over all its CTAs: 0 earliest kernel
 * entry, 1 latest entry, 2 / 3 latest / earliest "previous kernel finished", 4 latest digit planes
 * done, 5 latest first MMA, 6 latest accumulation retired, 7 latest flush done, 8 latest CTA end.
 * The caller sets words 0 and 3 of each group to the largest int64 and the rest to 0 beforehand.
 * NULL switches it off. */
void nvfp4_gemv_tc_probe(void* device_buffer);

/* W4A4 (both operands in the reference's block-16 E8M0 format).  No counterpart in the reference,
 * which is W4A16 throughout (its target GPU has no FP4 tensor cores; README.md names W4A4 as the
 * aim for GPUs that have them).
 * launch_nvfp4_gemm_fp4: out[m][t] (fp16, row pitch ld_out >= n_tokens) = dequant(W)[m][:] .
 *   dequant(A)[t][:], W = packed [M][K/2] + scales [M][K/16], A = packed [n_tokens][K/2] + scales
 *   [n_tokens][K/16].  Block-scaled FP4 tensor-core instruction (tcgen05.mma kind::mxf4nvf4, 16-element
 *   E8M0 scale blocks): the nibbles and scale bytes go to the tensor core as they are, fp32
 *   accumulation.  K % 256 == 0, all pointers 16-byte aligned.  0; -2 shape / pointer not taken;
 *   -3 no tensor-map encoder in the driver; else the launch's cudaError_t.
 * launch_nvfp4_quant_dequant_T: dst[k][t] = dequantise(quantise(src[t][:]))[k], the codec applied
 *   per token row along K, written token-minor (rows ld_dst >= n long, tail zeroed).
 * launch_nvfp4_gemm_w4a4: fp16 activations [n_tokens][K] in, out[M][N] (N = n_tokens rounded up to
 *   8).  work: K * N fp16 elements of scratch.  Activations are encoded with launch_nvfp4_encode
 *   into work and multiplied by launch_nvfp4_gemm_fp4; shapes that kernel does not take go through
 *   launch_nvfp4_quant_dequant_T and launch_nvfp4_gemmtc_v5 (fp16 holds every FP4 value times its
 *   power-of-two scale exactly, so both routes compute the same products; the second runs at the
 *   fp16 tensor rate).  0; -2 bad arguments; else a launch error.
 * nvfp4_gemm_fp4_status: like nvfp4_gemm_status, for the FP4 kernel's bounded waits alone
 *   (nvfp4_gemm_status reports them as 100 + id).
 * nvfp4_b200_gemm_fp4_config: bit 0: shapes whose output tiles would leave more than half of the SMs
 *   idle and whose K is deep (32 tokens x 5120 rows x K 17408: 40 tiles) split K over several CTAs per
 *   tile; the CTA that arrives last adds the fp32 partial tiles in split order (split launches on one
 *   device share a workspace and must follow one another in stream order).  Bit 1: more than 128
 *   tokens and K >= 10240 run on the CTA-pair kernel (clusters of two, tcgen05 cta_group::2, each
 *   CTA loading half of the token tile); bit 2: every K.  Bit 3: one CTA (pair) per output
 *   tile instead of one per SM (two SMs) that walks the tiles; bits 8..15: pairs of the walking pair
 *   kernel (0 = half the SM count).  Default 3.  Bit-identical results. */
void nvfp4_b200_gemm_fp4_config(int flags);
int launch_nvfp4_gemm_fp4(const uint8_t* w_packed, const uint8_t* w_scales, const uint8_t* a_packed,
                          const uint8_t* a_scales, void* out, int M, int n_tokens, int K, int ld_out,
                          void* stream);
int nvfp4_gemm_fp4_status(int reset);
int launch_nvfp4_quant_dequant_T(const void* src, long long ld_src, void* dst, long long ld_dst,
                                 int n, int K, void* stream);
int launch_nvfp4_gemm_w4a4(const uint8_t* d_weight_packed, const uint8_t* d_weight_scales,
                           const void* d_activation, void* d_output, void* work, int M,
                           int n_tokens, int K, void* stream);

/* The DeltaNet step without a caller-provided workspace.  It has no counterpart in the reference,
 * whose caller always allocates the scratch tensor itself.  It exists for callers that cannot
 * allocate device memory at the point of the call: code that runs after all device memory has
 * been given to another allocator, a plug-in that only receives its input and output buffers, or
 * code entered during stream capture, where cudaMalloc is not allowed.  The workspace is a 40 KB
 * array inside the library (every GPU that loads the library holds it until exit), so the shard
 * may have at most 10240 conv channels, (2 n_kheads + n_vheads) * 128 <= 10240 — the full model
 * exactly; beyond that the call prints a message and returns -2.  The array's device address is
 * looked up on the first call on each device: make that first call outside stream capture.
 * Calls on one device share the workspace and must not overlap on the GPU.  Arguments and results
 * otherwise as launch_dn_fused_heads, minus `scratch`. */
int launch_dn_fused_noalloc(const void* mixed, const void* z, const void* b, const void* a,
                            const void* conv_w, void* conv_state, const void* A_log,
                            const void* dt_bias, const void* norm_w, void* state, void* out,
                            int n_kheads, int n_vheads, float rms_eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H */

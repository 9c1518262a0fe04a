"""CPU oracle for one decode step of the hybrid decoder.  TEST INFRASTRUCTURE ONLY.

A numpy restatement of the model arithmetic the reference runs per generated token: the
third-party model's decoder layer (transformers Qwen3_5DecoderLayer: pre-norm token mixer +
residual, pre-norm gated MLP + residual) with every linear layer an NVFP4 GEMV and every
fused operator the reference substitutes (pipeline/_qwen38_infer.py:456-479 DeltaNet layer,
:612-644 gated attention layer, :856-903 RMSNorm; experiments/_qwen38_p9_fuse.py:48-116 RoPE and
silu*mul).  Built from ``fused_ops_oracle`` and ``nvfp4_codec_oracle``; a GEMV returns the
correctly rounded fp16 of the float64 product of the exactly decoded weights.

Parity status: UNPINNED at model level — the reference ships neither weights nor stored token
lists, and its acceptance tests compare two GPU stacks with each other.  The building blocks are
pinned (codec: golden vectors; fused operators: the reference's kernels run on the GPU).

Weights use the reference's names (``layers.{i}.self_attn.q_proj`` ...); see ``make_weights``.
Only tests, the smoke check and the CPU-baseline leg of the benchmark import this module.
"""
from __future__ import annotations

import numpy as np

from . import fused_ops_oracle as fo
from . import nvfp4_codec_oracle as oc

HEAD_DIM, DN_DIM, CONV_K = 256, 128, 4


def make_weights(cfg, seed: int, sigma: float = 0.02, norm_jitter: float = 0.1):
    """Seeded synthetic weights in the reference container's form: every linear weight
    ~N(0, sigma^2) fp16 encoded with the codec -> (packed, scales); norms, conv, A_log, dt_bias
    as fp16 arrays with the model's initialisation (zero-centred RMSNorm weights around 0, gated
    norm weights around 1, A_log = log U(0, 16), dt_bias = 1)."""
    rng = np.random.default_rng(seed)
    W = {}

    def lin(name, M, K):
        w = (rng.standard_normal((M, K), dtype=np.float32) * np.float32(sigma)).astype(np.float16)
        W[name] = oc.encode(w)

    def vec(name, n, center, jitter):
        W[name] = (center + jitter * rng.standard_normal(n)).astype(np.float16)

    for i in range(cfg.n_layers):
        pre = f"layers.{i}."
        for n, (M, K) in cfg.layer_shapes(i).items():
            sub = "mlp." if n in ("gate_proj", "up_proj", "down_proj") else \
                ("self_attn." if cfg.is_attn(i) else "linear_attn.")
            lin(pre + sub + n, M, K)
        vec(pre + "input_layernorm.weight", cfg.hidden, 0.0, norm_jitter)
        vec(pre + "post_attention_layernorm.weight", cfg.hidden, 0.0, norm_jitter)
        if cfg.is_attn(i):
            vec(pre + "self_attn.q_norm.weight", HEAD_DIM, 0.0, norm_jitter)
            vec(pre + "self_attn.k_norm.weight", HEAD_DIM, 0.0, norm_jitter)
        else:
            a = pre + "linear_attn."
            W[a + "conv1d.weight"] = (rng.standard_normal((cfg.conv_dim, CONV_K)) * 0.3).astype(np.float16)
            W[a + "A_log"] = np.log(rng.uniform(1e-3, 16, cfg.dn_vheads)).astype(np.float16)
            W[a + "dt_bias"] = np.ones(cfg.dn_vheads, dtype=np.float16)
            vec(a + "norm.weight", DN_DIM, 1.0, norm_jitter)
    W["embed_tokens"] = (rng.standard_normal((cfg.vocab, cfg.hidden)) * 0.5).astype(np.float16)
    vec("norm.weight", cfg.hidden, 0.0, norm_jitter)
    lin("lm_head", cfg.vocab, cfg.hidden)
    return W


class OracleModel:
    def __init__(self, cfg, weights, cos, sin):
        self.cfg, self.W = cfg, weights
        self.cos, self.sin = cos, sin
        self.dec = {}      # decoded float64 matrices, on demand
        self.reset()

    def reset(self):
        c = self.cfg
        self.pos = 0
        self.kv = {}
        self.dn = {}
        for i in range(c.n_layers):
            if c.is_attn(i):
                self.kv[i] = (np.zeros((c.hkv, c.max_len, HEAD_DIM), np.float16),
                              np.zeros((c.hkv, c.max_len, HEAD_DIM), np.float16))
            else:
                self.dn[i] = (np.zeros((c.conv_dim, CONV_K), np.float16),
                              np.zeros((c.dn_vheads, DN_DIM, DN_DIM), np.float32))

    def _w(self, name):
        if name not in self.dec:
            self.dec[name] = oc.decode_f64(*self.W[name])
        return self.dec[name]

    def gemv(self, name, x):
        with np.errstate(over="ignore"):
            return (self._w(name) @ np.asarray(x, np.float16).astype(np.float64)).astype(np.float16)

    def _w1(self, name):
        return (1.0 + np.asarray(self.W[name], np.float16).astype(np.float32)).astype(np.float32)

    @staticmethod
    def _add(a, b):
        return (np.asarray(a, np.float16).astype(np.float64) +
                np.asarray(b, np.float16).astype(np.float64)).astype(np.float16)

    def step(self, tok: int):
        """Process token `tok` at the current position; returns the fp16 logits."""
        c = self.cfg
        h = np.asarray(self.W["embed_tokens"][tok], np.float16)
        for i in range(c.n_layers):
            pre = f"layers.{i}."
            x = fo.rmsnorm(h[None], self._w1(pre + "input_layernorm.weight"), c.rms_eps)[0]
            if c.is_attn(i):
                a = pre + "self_attn."
                qg = self.gemv(a + "q_proj", x).reshape(c.hq, 2 * HEAD_DIM)
                q, gate = qg[:, :HEAD_DIM], qg[:, HEAD_DIM:]
                k = self.gemv(a + "k_proj", x).reshape(c.hkv, HEAD_DIM)
                v = self.gemv(a + "v_proj", x).reshape(c.hkv, HEAD_DIM)
                q = fo.rmsnorm(q, self._w1(a + "q_norm.weight"), c.rms_eps)
                k = fo.rmsnorm(k, self._w1(a + "k_norm.weight"), c.rms_eps)
                q = fo.rope_qk(q, self.cos[self.pos], self.sin[self.pos])
                k = fo.rope_qk(k, self.cos[self.pos], self.sin[self.pos])
                keys, vals = self.kv[i]
                keys[:, self.pos] = k
                vals[:, self.pos] = v
                o = fo.attn_decode(q, keys, vals, self.pos + 1, gate, HEAD_DIM ** -0.5,
                                   gqa=c.hq // c.hkv)
                mix = self.gemv(a + "o_proj", o.reshape(-1))
            else:
                a = pre + "linear_attn."
                mixed = self.gemv(a + "in_proj_qkv", x)
                z = self.gemv(a + "in_proj_z", x)
                b = self.gemv(a + "in_proj_b", x)
                al = self.gemv(a + "in_proj_a", x)
                conv_state, state = self.dn[i]
                o, conv_state, state, _ = fo.dn_fused_heads(
                    mixed, z, b, al, self.W[a + "conv1d.weight"], conv_state, self.W[a + "A_log"],
                    self.W[a + "dt_bias"], self.W[a + "norm.weight"], state, c.rms_eps,
                    c.dn_kheads, c.dn_vheads)
                self.dn[i] = (conv_state, state)
                mix = self.gemv(a + "out_proj", o)
            h = self._add(h, mix)
            x = fo.rmsnorm(h[None], self._w1(pre + "post_attention_layernorm.weight"), c.rms_eps)[0]
            m = pre + "mlp."
            act = fo.silu_mul(self.gemv(m + "gate_proj", x), self.gemv(m + "up_proj", x))
            h = self._add(h, self.gemv(m + "down_proj", act))
        x = fo.rmsnorm(h[None], self._w1("norm.weight"), c.rms_eps)[0]
        logits = self.gemv("lm_head", x)
        self.pos += 1
        return logits

    def run(self, prompt, n_gen: int):
        """Teacher-forced prompt, then greedy generation.  Returns (tokens, logits per generated
        token, top-1 minus top-2 margin per generated token)."""
        self.reset()
        logits = None
        for t in prompt:
            logits = self.step(int(t))
        toks, all_logits, margins = [], [], []
        for _ in range(n_gen):
            lf = logits.astype(np.float32)
            nxt = int(np.argmax(lf))
            top2 = np.partition(lf, -2)[-2:]
            toks.append(nxt)
            all_logits.append(logits)
            margins.append(float(top2[1] - top2[0]))
            if len(toks) < n_gen:
                logits = self.step(nxt)
        return toks, all_logits, margins


def make_weights_random_bytes(cfg, seed: int, norm_jitter: float = 0.1):
    """Like :func:`make_weights`, but every linear weight is drawn directly as NVFP4 bytes
    (uniform packed bytes, scale bytes uniform in [118, 122]: values of about the size
    N(0, 0.02^2) weights quantise to), so a full-width model can be built in seconds instead of
    being quantised on the CPU for minutes.  Any byte pattern is a valid NVFP4 matrix."""
    rng = np.random.default_rng(seed)
    W = {}

    def lin(name, M, K):
        W[name] = (rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8),
                   rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8))

    def vec(name, n, center, jitter):
        W[name] = (center + jitter * rng.standard_normal(n)).astype(np.float16)

    for i in range(cfg.n_layers):
        pre = f"layers.{i}."
        for n, (M, K) in cfg.layer_shapes(i).items():
            sub = "mlp." if n in ("gate_proj", "up_proj", "down_proj") else \
                ("self_attn." if cfg.is_attn(i) else "linear_attn.")
            lin(pre + sub + n, M, K)
        vec(pre + "input_layernorm.weight", cfg.hidden, 0.0, norm_jitter)
        vec(pre + "post_attention_layernorm.weight", cfg.hidden, 0.0, norm_jitter)
        if cfg.is_attn(i):
            vec(pre + "self_attn.q_norm.weight", HEAD_DIM, 0.0, norm_jitter)
            vec(pre + "self_attn.k_norm.weight", HEAD_DIM, 0.0, norm_jitter)
        else:
            a = pre + "linear_attn."
            W[a + "conv1d.weight"] = (rng.standard_normal((cfg.conv_dim, CONV_K)) * 0.3).astype(np.float16)
            W[a + "A_log"] = np.log(rng.uniform(1e-3, 16, cfg.dn_vheads)).astype(np.float16)
            W[a + "dt_bias"] = np.ones(cfg.dn_vheads, dtype=np.float16)
            vec(a + "norm.weight", DN_DIM, 1.0, norm_jitter)
    W["embed_tokens"] = (rng.standard_normal((cfg.vocab, cfg.hidden)) * 0.5).astype(np.float16)
    vec("norm.weight", cfg.hidden, 0.0, norm_jitter)
    lin("lm_head", cfg.vocab, cfg.hidden)
    return W

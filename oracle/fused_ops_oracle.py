"""CPU oracle for the fused decode-step operators.  TEST INFRASTRUCTURE ONLY.

numpy restatements of the operators the reference implements in
kernels/nvfp4_rmsnorm.cu, kernels/nvfp4_rope_silu.cu, kernels/nvfp4_attn_decode.cu and
kernels/nvfp4_dn_fused.cu.  Every place where the reference rounds a value to fp16 is rounded to
fp16 here too; everything between two rounding points is evaluated in float64, i.e. this oracle
returns the correctly rounded result of the reference's formula.  A CUDA kernel that evaluates
the same formula in fp32 therefore agrees bit-for-bit except where its fp32 intermediate lands
within an fp32 rounding error of an fp16 rounding boundary; the tests allow one fp16 ulp for that.

Parity status: the reference stores no golden vectors for these operators (its own checks are
relational: RMSNorm max-diff 0 against the model's module, experiments/_qwen38_p5b_attn.py:77-98;
a one-step DeltaNet A/B, pipeline/_qwen38_r2.py:163-185).  The oracle is pinned instead against
the reference kernels themselves, recompiled unchanged and run next to ours on the GPU
(``oracle/Makefile`` -> ``oracle/_ref``, ``tests/test_ref_kernels_gpu.py``), and against the
model's own PyTorch modules (the installed transformers Qwen3_5 code on the same dequantised
weights, ``tests/test_oracle_vs_hf.py``).

Only tests, the smoke check and the CPU-baseline leg of the benchmark import this module.
"""
from __future__ import annotations

import numpy as np

F16 = np.float16
F32 = np.float32
F64 = np.float64


def _r16(x):
    """Round to fp16 and return as float64 (an fp16 tensor store followed by a reload)."""
    with np.errstate(over="ignore"):
        return np.asarray(x).astype(F16).astype(F64)


def _r32(x):
    return np.asarray(x).astype(F32).astype(F64)


def rmsnorm(x: np.ndarray, w1: np.ndarray, eps: float) -> np.ndarray:
    """out = f16( f32(x) * rsqrt(mean(x^2) + eps) * w1 ), rows along the last axis.

    w1 is the precomputed fp32 (1 + weight).  Reference: kernels/nvfp4_rmsnorm.cu:39-61.
    """
    xf = np.asarray(x, dtype=F16).astype(F64)
    n = xf.shape[-1]
    ss = _r32((xf * xf).sum(axis=-1, keepdims=True))
    inv = _r32(1.0 / np.sqrt(_r32(_r32(ss / F64(n)) + F64(F32(eps)))))
    t = _r32(xf * inv)
    return _r32(t * np.asarray(w1, dtype=F32).astype(F64)).astype(F16)


def rope_qk(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x [heads, 256] fp16; cos/sin [256] fp16.  out = f16(f16(x*c) + f16(rot(x)*s)) with
    rot(x) = (-x2, x1).  Reference: kernels/nvfp4_rope_silu.cu:29-53."""
    xf = np.asarray(x, dtype=F16).astype(F64)
    c = np.asarray(cos, dtype=F16).astype(F64)
    s = np.asarray(sin, dtype=F16).astype(F64)
    half = xf.shape[-1] // 2
    rot = np.concatenate([-xf[..., half:], xf[..., :half]], axis=-1)
    return (_r16(xf * c) + _r16(rot * s)).astype(F16)


def silu(x64: np.ndarray) -> np.ndarray:
    return x64 / (1.0 + np.exp(-x64))


def silu_mul(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """out = f16( f32(f16(g / (1 + exp(-g)))) * f32(u) ).  Reference:
    kernels/nvfp4_rope_silu.cu:56-67."""
    gf = np.asarray(g, dtype=F16).astype(F64)
    uf = np.asarray(u, dtype=F16).astype(F64)
    return (_r16(silu(gf)) * uf).astype(F16)


def attn_decode(q, keys, values, L, gate, scale, gqa=6):
    """GQA decode attention with sigmoid output gate.

    q [HQ, D], keys/values [HKV, max_len, D], gate [HQ, D], all fp16; L keys are valid.
    scores = (q.k) * scale in fp32 -> softmax -> o = sum p v -> f16(f16(o) * f16(sigmoid(gate))).
    Reference: kernels/nvfp4_attn_decode.cu:50-117.
    """
    q = np.asarray(q, dtype=F16).astype(F64)
    gate = np.asarray(gate, dtype=F16).astype(F64)
    HQ, D = q.shape
    out = np.empty((HQ, D), dtype=F16)
    for h in range(HQ):
        kv = h // gqa
        k = np.asarray(keys[kv, :L], dtype=F16).astype(F64)
        v = np.asarray(values[kv, :L], dtype=F16).astype(F64)
        s = _r32(_r32(k @ q[h]) * F64(F32(scale)))
        m = s.max()
        e = _r32(np.exp(_r32(s - m)))
        p = _r32(e * _r32(1.0 / _r32(e.sum())))
        o = p @ v
        sg = _r16(1.0 / (1.0 + np.exp(-gate[h])))
        out[h] = (_r16(o) * sg).astype(F16)
    return out


def softplus(x64):
    return np.where(x64 > 20.0, x64, np.log1p(np.exp(np.minimum(x64, 20.0))))


def dn_conv(mixed, conv_w, conv_state):
    """Causal conv1d update (kernel 4) + silu for every channel.

    mixed [C] fp16, conv_w [C, 4] fp16, conv_state [C, 4] fp16 (layout c*4 + t).
    Returns (scratch float32 [C] holding fp16-rounded values, new_state fp16 [C, 4]).
    Window is [s1, s2, s3, x]; the oldest frame s0 is dropped.
    Reference: kernels/nvfp4_dn_fused.cu:55-76.
    """
    x = np.asarray(mixed, dtype=F16)
    w = np.asarray(conv_w, dtype=F16).reshape(-1, 4).astype(F64)
    st = np.asarray(conv_state, dtype=F16).reshape(-1, 4)
    win = np.concatenate([st[:, 1:], x[:, None]], axis=1)
    acc = _r32((w * win.astype(F64)).sum(axis=1))
    return _r16(silu(acc)).astype(F32), win.copy()


def dn_rec(scratch, z, b, a, A_log, dt_bias, norm_w, state, rms_eps,
           n_vheads=48, n_kheads=16, dk=128):
    """Gated delta rule recurrent step + RMSNormGated.

    scratch float32 [2*KEY + VAL] = conv output [q | k | v]; state float32 [NVH, dk(v row j), dk(i)]
    (transposed: row j of a head is the state column of value dim j).
    Returns (out fp16 [NVH*dk], new_state float32).
    Reference: kernels/nvfp4_dn_fused.cu:96-152.
    """
    key_dim = n_kheads * dk
    rep = n_vheads // n_kheads
    sc = np.asarray(scratch, dtype=F32).astype(F64)
    S = np.asarray(state, dtype=F32).reshape(n_vheads, dk, dk).astype(F64)
    z = np.asarray(z, dtype=F16).astype(F64).reshape(n_vheads, dk)
    nw = np.asarray(norm_w, dtype=F16).astype(F64)
    out = np.empty((n_vheads, dk), dtype=F16)
    newS = np.empty((n_vheads, dk, dk), dtype=F32)
    for h in range(n_vheads):
        kh = h // rep
        beta = _r16(1.0 / (1.0 + np.exp(-F64(F16(b[h])))))
        g = _r32(-_r32(np.exp(F64(F16(A_log[h])))) *
                 _r32(softplus(_r32(F64(F16(a[h])) + F64(F16(dt_bias[h]))))))
        eg = _r32(np.exp(g))
        qv = sc[kh * dk:(kh + 1) * dk]
        kv = sc[key_dim + kh * dk:key_dim + (kh + 1) * dk]
        inv_q = _r32(_r32(1.0 / np.sqrt(_r32(_r32((qv * qv).sum()) + F64(F32(1e-6))))) *
                     F64(F32(0.08838834764831845)))
        inv_k = _r32(1.0 / np.sqrt(_r32(_r32((kv * kv).sum()) + F64(F32(1e-6)))))
        qn = _r32(qv * inv_q)
        kn = _r32(kv * inv_k)
        v = sc[2 * key_dim + h * dk:2 * key_dim + (h + 1) * dk]
        Sd = _r32(S[h] * eg)                       # decayed state, [j, i]
        kvp = _r32(Sd @ kn)                        # [j]
        delta = _r32(_r32(v - kvp) * beta)         # [j]
        Sn = _r32(Sd + kn[None, :] * delta[:, None])
        newS[h] = Sn.astype(F32)
        o = _r16(Sn @ qn)                          # [j], rounded to fp16
        var = _r32(_r32((o * o).sum()) / F64(dk))
        xn = _r32(o * _r32(1.0 / np.sqrt(_r32(var + F64(F32(rms_eps))))))
        hw = _r16(_r16(xn) * nw)                   # fp16 multiply
        out[h] = _r32(hw * _r32(silu(z[h]))).astype(F16)
    return out.reshape(-1), newS


def dn_fused(mixed, z, b, a, conv_w, conv_state, A_log, dt_bias, norm_w, state, rms_eps):
    """One Gated-DeltaNet decode step = dn_conv followed by dn_rec.
    Returns (out fp16 [6144], new_conv_state fp16 [C,4], new_state float32, scratch float32)."""
    scratch, new_conv = dn_conv(mixed, conv_w, conv_state)
    out, new_state = dn_rec(scratch, z, b, a, A_log, dt_bias, norm_w, state, rms_eps)
    return out, new_conv, new_state, scratch


def dn_fused_heads(mixed, z, b, a, conv_w, conv_state, A_log, dt_bias, norm_w, state, rms_eps,
                   n_kheads, n_vheads):
    """dn_fused for a shard / model with n_kheads key heads and n_vheads value heads."""
    scratch, new_conv = dn_conv(mixed, conv_w, conv_state)
    out, new_state = dn_rec(scratch, z, b, a, A_log, dt_bias, norm_w, state, rms_eps,
                            n_vheads=n_vheads, n_kheads=n_kheads)
    return out, new_conv, new_state, scratch

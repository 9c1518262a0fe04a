"""Generate tests/golden/codec_golden.npz by importing the reference's own Python codec.

Run once, in a checkout that has the reference mounted:

    python tests/golden/make_golden.py <reference checkout>

The reference tree is only read (its ``codec/`` directory is put on ``sys.path``); nothing is
copied from it.  The resulting ``.npz`` travels with the repository, so the tests that use it
need neither the reference nor a GPU.

Contents (all arrays produced by reference functions, names in brackets):
  edge_in / edge_packed / edge_scales / edge_dec   the seven 1x16 edge cases of the reference's
        self-test [encode_fp16_to_nvfp4, decode_nvfp4_to_fp16]
  m{i}_in / m{i}_packed / m{i}_scales / m{i}_dec   random matrices, encoded with the reference's
        loop encoder (small) or its vectorised twin (large) and decoded with its loop decoder
  scale_all   scale byte for every non-negative finite fp16 block maximum [compute_block_scale]
  code_all    E2M1 code for every non-negative finite fp16 value times 2^e, e in [-6, 6]
        [fp32_to_e2m1_code]
  emb_idx / emb_rows   rows decoded by the reference's vectorised decoder (PackedEmb arithmetic:
        nibble LUT x exp2(scale-127) in fp64 -> fp16)
  gemv_*      a small GEMV: y = decode(packed, scales).astype(f32) @ act.astype(f32)
        (the reference's truth recipe)
"""
from __future__ import annotations

import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "codec"))
    import nvfp4_codec as ref  # noqa: E402
    import nvfp4_codec_fast as ref_fast  # noqa: E402

    out = {}

    # ---- the reference's edge cases (codec/nvfp4_codec.py:430-439) ----
    edge = [
        np.zeros((1, 16), dtype=np.float16),
        np.full((1, 16), 6.0, dtype=np.float16),
        np.full((1, 16), -6.0, dtype=np.float16),
        np.full((1, 16), 100.0, dtype=np.float16),
        np.full((1, 16), 0.001, dtype=np.float16),
        np.full((1, 16), -0.0, dtype=np.float16),
        np.array([[1.5, -3.0, 0.5, -0.0, 6.0, -6.0, 2.0, -1.0,
                   4.0, -4.0, 0.0, -0.5, 3.0, -1.5, 5.0, -2.5]], dtype=np.float16),
    ]
    e_in = np.concatenate(edge, axis=0)
    e_p, e_s, e_d = [], [], []
    for m in edge:
        p, s = ref.encode_fp16_to_nvfp4(m)
        e_p.append(p)
        e_s.append(s)
        e_d.append(ref.decode_nvfp4_to_fp16(p, s))
    out["edge_in"] = e_in
    out["edge_packed"] = np.concatenate(e_p)
    out["edge_scales"] = np.concatenate(e_s)
    out["edge_dec"] = np.concatenate(e_d)

    # ---- random matrices ----
    rng = np.random.default_rng(7)
    mats = [
        (rng.standard_normal((16, 64)) * 2.0).astype(np.float16),
        (rng.standard_normal((24, 256)) * 0.3).astype(np.float16),
        np.hstack([rng.standard_normal((8, 128)) * 1e-3,
                   rng.standard_normal((8, 128)) * 1e3]).astype(np.float16),
        (rng.standard_normal((12, 96)) * 0.02).astype(np.float16),
        # values that sit exactly on rounding midpoints after normalisation
        (rng.choice(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 0.0, -0.75, -3.5]),
                    size=(8, 64))).astype(np.float16),
        # huge and tiny magnitudes, inf-free
        np.clip(rng.standard_normal((4, 64)) * rng.choice([6e-8, 1e-5, 1.0, 3e4], (4, 64)),
                -65504.0, 65504.0).astype(np.float16),
    ]
    for i, m in enumerate(mats):
        p, s = ref.encode_fp16_to_nvfp4(m)
        pf, sf = ref_fast.encode_fp16_to_nvfp4_fast(m)
        assert np.array_equal(p, pf) and np.array_equal(s, sf)
        out[f"m{i}_in"] = m
        out[f"m{i}_packed"] = p
        out[f"m{i}_scales"] = s
        out[f"m{i}_dec"] = ref.decode_nvfp4_to_fp16(p, s)
    out["n_mats"] = np.array(len(mats))

    # ---- exhaustive scale rule: every non-negative finite fp16 as the block maximum ----
    bits = np.arange(0, 0x7C00, dtype=np.uint16)
    vals = bits.view(np.float16)
    out["scale_all"] = np.array(
        [ref.compute_block_scale(np.array([v], dtype=np.float16)) for v in vals], dtype=np.uint8)

    # ---- exhaustive rounding rule ----
    exps = np.arange(-6, 7)
    codes = np.empty((len(exps), len(vals)), dtype=np.uint8)
    v64 = vals.astype(np.float64)
    for j, e in enumerate(exps):
        codes[j] = ref.fp32_to_e2m1_code((v64 * 2.0 ** e).astype(np.float32))
    out["code_exps"] = exps
    out["code_all"] = codes

    # ---- the reference's vectorised decoder arithmetic (pipeline/_qwen38_infer.py:114-127) ----
    w = (rng.standard_normal((40, 128)) * 0.05).astype(np.float16)
    p, s = ref_fast.encode_fp16_to_nvfp4_fast(w)
    lut = (np.where(np.arange(16) & 8, -1.0, 1.0) * ref.E2M1_ABS_CODEPOINTS[np.arange(16) & 7]).astype(np.float32)
    idx = np.array([0, 3, 39, 17], dtype=np.int64)
    pp, sb = p[idx], s[idx]
    nib = np.empty((len(idx), pp.shape[1] * 2), dtype=np.uint8)
    nib[:, 0::2] = pp & 0x0F
    nib[:, 1::2] = pp >> 4
    wv = lut[nib].reshape(len(idx), -1, 16)
    sc = np.exp2(sb.astype(np.float64) - 127.0)
    out["emb_packed"] = p
    out["emb_scales"] = s
    out["emb_idx"] = idx
    out["emb_rows"] = (wv * sc[:, :, None]).astype(np.float16).reshape(len(idx), -1)

    # ---- a small GEMV with the reference's truth recipe ----
    W = (rng.standard_normal((48, 256)) * 0.02).astype(np.float16)
    a = rng.standard_normal(256).astype(np.float16)
    p, s = ref.encode_fp16_to_nvfp4(W)
    out["gemv_packed"] = p
    out["gemv_scales"] = s
    out["gemv_act"] = a
    out["gemv_y_f32"] = ref.decode_nvfp4_to_fp16(p, s).astype(np.float32) @ a.astype(np.float32)

    # ---- calibrated-matrix quality figures (codec/nvfp4_codec.py:282-421, seed 42, 16x16) ----
    r2 = np.random.default_rng(42)
    cal = (r2.standard_normal((16, 16)) * 0.3).astype(np.float16)
    p, s = ref.encode_fp16_to_nvfp4(cal)
    d = ref.decode_nvfp4_to_fp16(p, s)
    out["cal_in"] = cal
    out["cal_dec"] = d

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "codec_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])

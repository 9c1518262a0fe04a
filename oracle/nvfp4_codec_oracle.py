"""CPU oracle for the NVFP4 codec and the GEMV / GEMM built on it.  TEST INFRASTRUCTURE ONLY.

This module is a numpy restatement of the reference's CPU algorithm.  It is imported by the test
suite, by the smoke check and by the CPU-baseline leg of the benchmark, and by nothing else: the
shipped library never calls it.

Parity status: PINNED.  ``tests/golden/codec_golden.npz`` holds inputs and outputs produced by
importing the reference's own ``codec/nvfp4_codec.py`` and ``codec/nvfp4_codec_fast.py`` (script:
``tests/golden/make_golden.py``); ``tests/test_oracle_codec.py`` checks every function below
against those vectors, against the reference's seven edge-case known answers
(scale bytes 127/127/127/132/115/127/127) and against its calibrated-matrix quality figures
(cosine 0.9926, SNR 18.3 dB).

Format (reference: codec/nvfp4_codec.py:41-59,92-125,166-200):
  element : E2M1 nibble = sign<<3 | code, code -> {0, .5, 1, 1.5, 2, 3, 4, 6}
  packing : byte i of a row = element 2i (low nibble) | element 2i+1 (high nibble) << 4
  scale   : one byte per 16 consecutive elements of a row, value 2^(byte-127)
"""
from __future__ import annotations

import numpy as np

E2M1_ABS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_MAX = 6.0
BLOCK = 16
BIAS = 127
# midpoints between neighbouring code points; a value exactly on a midpoint takes the SMALLER code
# (reference: argmin returns the first minimum, codec/nvfp4_codec.py:78-79; the packer states the
# same rule with searchsorted(side="left"), pipeline/_qwen38_nvfp4_pack.py:43-50)
E2M1_EDGES = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)

# nibble -> signed fp32 value (reference: pipeline/_qwen38_infer.py:114-115)
NIBBLE_LUT = (np.where(np.arange(16) & 8, -1.0, 1.0) * E2M1_ABS[np.arange(16) & 7]).astype(np.float32)


def block_scale_bytes(max_abs: np.ndarray) -> np.ndarray:
    """Per-block max |x| (float64) -> E8M0 byte.

    exponent = ceil(log2(max/6)) clipped to [-127, 127]; an all-zero block gets exponent 0
    (byte 127).  Reference: codec/nvfp4_codec.py:166-193.
    """
    max_abs = np.asarray(max_abs, dtype=np.float64)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.ceil(np.log2(max_abs / E2M1_MAX))
    e = np.where(max_abs > 0.0, e, 0.0)
    e = np.clip(e, -127.0, 127.0)
    return (e + BIAS).astype(np.uint8)


def e2m1_codes(abs_norm: np.ndarray) -> np.ndarray:
    """|x|/scale (float32) -> 3-bit code, round to nearest, ties to the smaller code.

    Reference: codec/nvfp4_codec.py:62-80 (clip to [0, 6], argmin over the 8 code points).
    """
    a = np.clip(np.asarray(abs_norm, dtype=np.float32), 0.0, E2M1_MAX)
    return np.searchsorted(E2M1_EDGES, a, side="left").astype(np.uint8)


def encode(fp16_matrix: np.ndarray, row_chunk: int = 4096):
    """fp16 [M, K] (K % 16 == 0) -> (packed u8 [M, K/2], scales u8 [M, K/16]).

    Reference: codec/nvfp4_codec.py:207-245 — scale from the fp64 block maximum, division in
    fp64 rounded to fp32, nearest code, -0 stored as +0.
    """
    assert fp16_matrix.dtype == np.float16 and fp16_matrix.ndim == 2
    M, K = fp16_matrix.shape
    assert K % BLOCK == 0
    nb = K // BLOCK
    packed = np.empty((M, K // 2), dtype=np.uint8)
    scales = np.empty((M, nb), dtype=np.uint8)
    for r0 in range(0, M, row_chunk):
        r1 = min(M, r0 + row_chunk)
        x = fp16_matrix[r0:r1].astype(np.float64).reshape(r1 - r0, nb, BLOCK)
        sb = block_scale_bytes(np.abs(x).max(axis=-1))
        scales[r0:r1] = sb
        sc = np.exp2(sb.astype(np.float64) - BIAS)
        norm = (x / sc[..., None]).astype(np.float32).reshape(r1 - r0, K)
        code = e2m1_codes(np.abs(norm))
        sign = (norm < 0).astype(np.uint8)  # -0.0 < 0 is False, so -0 -> +0
        nib = (sign << 3) | code
        packed[r0:r1] = (nib[:, 0::2] & 0x0F) | ((nib[:, 1::2] & 0x0F) << 4)
    return packed, scales


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    """packed u8 [..., K/2] -> nibbles u8 [..., K] (element order)."""
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0x0F
    out[..., 1::2] = packed >> 4
    return out


def decode_f64(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """(packed, scales) -> exact dequantised values as float64 [M, K].

    Reference: codec/nvfp4_codec.py:248-272 (fp64 intermediate).
    """
    M, Kh = packed.shape
    K = Kh * 2
    assert scales.shape == (M, K // BLOCK)
    w = NIBBLE_LUT[unpack_nibbles(packed)].astype(np.float64).reshape(M, K // BLOCK, BLOCK)
    sc = np.exp2(scales.astype(np.float64) - BIAS)
    return (w * sc[:, :, None]).reshape(M, K)


def decode(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """(packed, scales) -> fp16 [M, K].  Reference: codec/nvfp4_codec.py:248-275."""
    with np.errstate(over="ignore"):
        return decode_f64(packed, scales).astype(np.float16)


def byte_to_half_bits() -> np.ndarray:
    """All 256 packed bytes -> (low-nibble fp16 bits, high-nibble fp16 bits), uint16 [256, 2].

    Reference bit patterns: kernels/nvfp4_gemv.cu:37-40,52-54 (code 0 -> 0x0000, 1 -> 0x3800,
    c >= 2 -> 0x3800 + (c << 9); sign -> bit 15).
    """
    b = np.arange(256, dtype=np.uint32)

    def nib(n):
        c = n & 7
        mag = np.where(c >= 2, 0x3800 + (c << 9), np.where(c == 1, 0x3800, 0))
        return (mag | ((n & 8) << 12)).astype(np.uint16)

    return np.stack([nib(b & 0xF), nib(b >> 4)], axis=1)


def gemv_f64(packed: np.ndarray, scales: np.ndarray, act: np.ndarray) -> np.ndarray:
    """Truth column: float64 product of the exactly decoded matrix with fp16 activations.

    ``act`` is [K] or [T, K]; returns [M] or [T, M] float64.
    """
    w = decode_f64(packed, scales)
    a = np.asarray(act, dtype=np.float16).astype(np.float64)
    return (a @ w.T) if a.ndim == 2 else (w @ a)


def gemv_ref_f32(packed: np.ndarray, scales: np.ndarray, act: np.ndarray) -> np.ndarray:
    """The reference's own truth recipe: decode to fp16, then an fp32 matmul
    (simulation/nvfp4_cuda_v5_test.py:90-91)."""
    w = decode(packed, scales).astype(np.float32)
    a = np.asarray(act, dtype=np.float16).astype(np.float32)
    return (a @ w.T) if a.ndim == 2 else (w @ a)


def rel_error_floored(y: np.ndarray, ref: np.ndarray, floor_frac: float = 1e-3) -> np.ndarray:
    """|y - ref| / max(|ref|, floor_frac * max|ref|): relative error that does not blow up where
    the reference cancels to (almost) zero."""
    ref = np.asarray(ref, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    den = np.maximum(np.abs(ref), floor_frac * np.abs(ref).max())
    return np.abs(y - ref) / den


def reference_gemm_check(y: np.ndarray, ref: np.ndarray):
    """The reference's GEMM acceptance rule (simulation/nvfp4_cuda_v5_test.py:92-95):
    mean_rel < 0.01 and max_abs < max(0.1, 1 % of max|ref|), rel = err / (|ref| + 1e-3)."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    err = np.abs(y - ref)
    mean_rel = float((err / (np.abs(ref) + 1e-3)).mean())
    max_abs = float(err.max())
    ok = mean_rel < 0.01 and max_abs < max(0.1, 0.01 * float(np.abs(ref).max()))
    return ok, mean_rel, max_abs


def synthetic_weight(M: int, K: int, seed: int, sigma: float = 0.02) -> np.ndarray:
    """Seeded fp16 weight matrix ~N(0, sigma^2) (the benchmark configurations' distribution)."""
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((M, K), dtype=np.float32) * np.float32(sigma)).astype(np.float16)


def synthetic_act(K: int, seed: int, T: int | None = None) -> np.ndarray:
    rng = np.random.default_rng(seed + 1_000_003)
    shape = (K,) if T is None else (T, K)
    return rng.standard_normal(shape, dtype=np.float32).astype(np.float16)

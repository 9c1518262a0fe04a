"""Container writer: fp16 state dict -> ``nvfp4_packed.bin`` + ``nvfp4_index.json`` +
``fp16_embed.npy`` + ``fp32_misc.npz``, the on-disk format the decode engine bridge loads
(reference: pipeline/_qwen38_nvfp4_pack.py:95-133 for the layout, :34-67 for the quantiser).

Every 2-D tensor except the embedding is quantised row-wise and written as its packed bytes
immediately followed by its scale bytes; the index records ``{M, K, packed_off, packed_bytes,
scales_off, scales_bytes, fmt}`` per tensor name; non-2-D tensors go to ``fp32_misc.npz``.  The
reference reads sharded safetensors of a real checkpoint; here the source is any mapping
name -> array (synthetic weights), so a container can be produced without the checkpoint.

The quantiser below produces the reference's bytes by exact arithmetic instead of logarithms
and table searches (``tests/test_oracle_codec.py`` compares it with the golden vectors): it is the
host statement of what ``launch_nvfp4_encode`` does on the device.
  scale : the block maximum is m * 2^x with 0.5 <= m < 1 (``frexp``, exact); the smallest e with
          6 * 2^e >= max is x - 3 when m <= 0.75 and x - 2 otherwise; byte = e + 127; an all-zero
          block gets e = 0; e is clipped to [-127, 127].
  code  : |value| * 2^-e (exact) is compared with the seven midpoints between code points; the
          code is the number of midpoints strictly below it, so a value on a midpoint takes the
          smaller code.  The sign bit is set for values below zero only (-0 stores as +0).
This is an offline tool, not part of the GPU hot path.
"""
from __future__ import annotations

import json
import os

import numpy as np

E2M1_MAX_ABS = 6.0
BLOCK = 16
BIAS = 127
ROW_CHUNK = 4096
FMT = "nvfp4_v2_embedded_sign"
_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def encode_block_scales(max_abs_f64: np.ndarray):
    """Block maxima -> (scale bytes uint8, scale exponents float64)."""
    peak = np.asarray(max_abs_f64, dtype=np.float64)
    mant, expo = np.frexp(peak)
    e = expo - np.where(mant <= 0.75, 3, 2)
    e = np.where(peak > 0.0, e, 0)
    e = np.where(np.isinf(peak), 127, e)
    e = np.clip(e, -127, 127)
    return (e + BIAS).astype(np.uint8), e.astype(np.float64)


def e2m1_codes_rtn(abs_x: np.ndarray) -> np.ndarray:
    """|normalised value| -> 3-bit code, nearest code point, a tie goes to the smaller code."""
    a = np.asarray(abs_x)
    code = np.zeros(a.shape, dtype=np.uint8)
    for mid in _MIDPOINTS:
        code += a > mid
    return code


def encode_rows(w_f32: np.ndarray):
    """(rows, K) float32 -> packed (rows, K/2) uint8, scale bytes (rows, K/16) uint8."""
    rows, K = w_f32.shape
    if K % BLOCK:
        raise ValueError(f"K = {K} is not a multiple of {BLOCK}")
    blk = np.asarray(w_f32, dtype=np.float64).reshape(rows, K // BLOCK, BLOCK)
    sbytes, e = encode_block_scales(np.abs(blk).max(axis=2))
    unit = np.ldexp(blk, -e.astype(np.int64)[..., None]).astype(np.float32).reshape(rows, K)
    nibble = e2m1_codes_rtn(np.abs(unit)) | ((unit < 0).astype(np.uint8) << 3)
    pairs = nibble.reshape(rows, K // 2, 2)
    return pairs[..., 0] | (pairs[..., 1] << 4), sbytes


def encode_rows_device(w16, device="cuda"):
    """fp16 matrix (numpy array or torch tensor) -> (packed, scales) numpy arrays, quantised by
    ``launch_nvfp4_encode`` on the GPU: the same bytes as :func:`encode_rows`, at memory speed."""
    import ctypes

    import torch

    from .. import _lib

    lib = _lib.load()
    t = torch.as_tensor(w16).to(device=device, dtype=torch.float16).contiguous()
    M, K = t.shape
    packed = torch.empty((M, K // 2), dtype=torch.uint8, device=t.device)
    scales = torch.empty((M, K // BLOCK), dtype=torch.uint8, device=t.device)
    rc = lib.launch_nvfp4_encode(ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(packed.data_ptr()),
                                 ctypes.c_void_p(scales.data_ptr()), M, K,
                                 ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"launch_nvfp4_encode rc={rc}")
    return packed.cpu().numpy(), scales.cpu().numpy()


def pack_tensors(tensors: dict, out_dir: str, prequantised: dict | None = None,
                 device: str | None = None) -> dict:
    """Write a container.  ``tensors``: name -> numpy array (checkpoint naming, e.g.
    ``model.language_model.layers.0.mlp.gate_proj.weight``).  ``prequantised``: name ->
    (packed, scales) for matrices that are already in NVFP4 form.  ``device``: quantise on that
    GPU instead of the host.  Returns the index."""
    os.makedirs(out_dir, exist_ok=True)
    index, misc = {}, {}
    prequantised = prequantised or {}
    with open(os.path.join(out_dir, "nvfp4_packed.bin"), "wb") as out:
        for name in sorted(set(tensors) | set(prequantised)):
            if name.startswith("model.visual.") or "mtp" in name.lower():
                continue
            if name in prequantised:
                packed, scales = prequantised[name]
                M, K = packed.shape[0], packed.shape[1] * 2
            else:
                t = np.asarray(tensors[name])
                if t.ndim != 2:
                    misc[name] = t.astype(np.float32)
                    continue
                if "embed_tokens" in name:
                    np.save(os.path.join(out_dir, "fp16_embed.npy"), t.astype(np.float16))
                    continue
                M, K = t.shape
                w = t.astype(np.float16)
                if device is not None:
                    packed, scales = encode_rows_device(w, device)
                else:
                    parts = [encode_rows(w[r0:r0 + ROW_CHUNK].astype(np.float32))
                             for r0 in range(0, M, ROW_CHUNK)]
                    packed = np.concatenate([p for p, _ in parts])
                    scales = np.concatenate([s for _, s in parts])
            off_p = out.tell()
            out.write(np.ascontiguousarray(packed).tobytes())
            off_s = out.tell()
            out.write(np.ascontiguousarray(scales).tobytes())
            index[name] = {"M": int(M), "K": int(K), "packed_off": off_p,
                           "packed_bytes": int(packed.nbytes), "scales_off": off_s,
                           "scales_bytes": int(scales.nbytes), "fmt": FMT}
    np.savez(os.path.join(out_dir, "fp32_misc.npz"), **misc)
    with open(os.path.join(out_dir, "nvfp4_index.json"), "w", encoding="utf-8") as f:
        json.dump(index, f, indent=1)
    return index

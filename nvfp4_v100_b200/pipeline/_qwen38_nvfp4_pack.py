"""Container writer: fp16 state dict -> ``nvfp4_packed.bin`` + ``nvfp4_index.json`` +
``fp16_embed.npy`` + ``fp32_misc.npz``, the on-disk format the decode engine bridge loads.

Mirrors the reference's offline packer (pipeline/_qwen38_nvfp4_pack.py:34-67 quantiser,
:95-133 container layout): every 2-D tensor except the embedding is quantised row-wise (block max
in float64 -> scale exponent ceil(log2(max/6)) clipped to +-127, normalise in float64 -> float32,
nearest E2M1 code with ties to the smaller code, -0 stored as +0, two nibbles per byte) and
written as its packed bytes immediately followed by its scale bytes; the index records
``{M, K, packed_off, packed_bytes, scales_off, scales_bytes, fmt}`` per tensor name; non-2-D
tensors go to ``fp32_misc.npz``.  The reference reads sharded safetensors of a real checkpoint;
here the source is any mapping name -> array (synthetic weights), so a container can be produced
without the checkpoint.  This is an offline CPU tool, not part of the GPU hot path.
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
_EDGES = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


def encode_block_scales(max_abs_f64: np.ndarray):
    with np.errstate(divide="ignore", invalid="ignore"):
        scale_exp = np.ceil(np.log2(max_abs_f64 / E2M1_MAX_ABS))
    scale_exp = np.where(max_abs_f64 == 0.0, 0.0, scale_exp)
    scale_exp = np.clip(scale_exp, -127, 127)
    return (scale_exp + BIAS).astype(np.uint8), scale_exp


def e2m1_codes_rtn(abs_x: np.ndarray) -> np.ndarray:
    return np.searchsorted(_EDGES, np.clip(abs_x, 0.0, 6.0), side="left").astype(np.uint8)


def encode_rows(w_f32: np.ndarray):
    """(rows, K) float32 -> packed (rows, K/2) uint8, scale bytes (rows, K/16) uint8."""
    M, K = w_f32.shape
    assert K % BLOCK == 0
    blocks = w_f32.reshape(M, K // BLOCK, BLOCK)
    max_abs = np.abs(blocks).max(axis=-1).astype(np.float64)
    sbytes, sexp = encode_block_scales(max_abs)
    norm = (blocks / np.exp2(sexp)[..., None]).astype(np.float32).reshape(M, K)
    signs = (norm < 0).astype(np.uint8)
    nib = (signs << 3) | e2m1_codes_rtn(np.abs(norm))
    return (nib[:, 0::2] & 0x0F) | ((nib[:, 1::2] & 0x0F) << 4), sbytes


def pack_tensors(tensors: dict, out_dir: str, prequantised: dict | None = None) -> dict:
    """Write a container.  ``tensors``: name -> numpy array (checkpoint naming, e.g.
    ``model.language_model.layers.0.mlp.gate_proj.weight``).  ``prequantised``: name ->
    (packed, scales) for matrices that are already in NVFP4 form.  Returns the index."""
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

"""Helpers for the GPU parity tests: move numpy data to the device with torch (plumbing only)
and call the C ABI with raw pointers, exactly as a ctypes client of the reference DLLs does."""
import ctypes

import numpy as np
import torch


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def gemv(lib, packed: np.ndarray, scales: np.ndarray, act: np.ndarray, entry="launch_nvfp4_gemv_v8"):
    M, K = packed.shape[0], packed.shape[1] * 2
    d_p, d_s, d_a = dev(packed), dev(scales), dev(act.astype(np.float16))
    out = torch.full((M + 8,), float("nan"), dtype=torch.float16, device="cuda")  # canary tail
    rc = getattr(lib, entry)(ptr(d_p), ptr(d_s), ptr(d_a), ptr(out), M, K, stream())
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.isnan(o[M:]).all(), "kernel wrote past the end of the output"
    return rc, o[:M]


def gemv2(lib, packed, scales, act0, act1):
    M, K = packed.shape[0], packed.shape[1] * 2
    d_p, d_s = dev(packed), dev(scales)
    d_a0, d_a1 = dev(act0.astype(np.float16)), dev(act1.astype(np.float16))
    out = torch.full((2 * M + 8,), float("nan"), dtype=torch.float16, device="cuda")
    rc = lib.launch_nvfp4_gemv2(ptr(d_p), ptr(d_s), ptr(d_a0), ptr(d_a1), ptr(out), M, K, stream())
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.isnan(o[2 * M:]).all()
    return rc, o[:2 * M].reshape(2, M)


def gemv2i(lib, packed, scales, act0, act1):
    """launch_nvfp4_gemv2i: the two activations travel as K (a0[k], a1[k]) pairs."""
    M, K = packed.shape[0], packed.shape[1] * 2
    d_p, d_s = dev(packed), dev(scales)
    inter = np.stack([act0.astype(np.float16), act1.astype(np.float16)], axis=1).reshape(-1)
    d_a = dev(np.ascontiguousarray(inter))
    out = torch.full((2 * M + 8,), float("nan"), dtype=torch.float16, device="cuda")
    rc = lib.launch_nvfp4_gemv2i(ptr(d_p), ptr(d_s), ptr(d_a), ptr(out), M, K, stream())
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.isnan(o[2 * M:]).all()
    return rc, o[:2 * M].reshape(2, M)


def ulp_diff_f16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in fp16 representable steps between two fp16 arrays (sign-magnitude aware)."""
    def key(x):
        u = np.asarray(x, dtype=np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a) - key(b))

"""ctypes binding of ``libnvfp4_b200.so`` — the one C-ABI library behind every reference DLL name.

There is no fallback: if the library is missing, or does not export a symbol the header declares,
loading raises.  Signatures follow ``include/nvfp4_b200.h``.
"""
from __future__ import annotations

import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libnvfp4_b200.so")
KDIR = os.path.join(PKG_DIR, "kernels")

_vp, _i, _f, _sz, _ll = (ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t,
                         ctypes.c_longlong)

_GEMV_SIG = ([_vp, _vp, _vp, _vp, _i, _i, _vp], _i)

# symbol -> (argtypes, restype); mirrors include/nvfp4_b200.h
SIGNATURES = {
    "gpu_malloc": ([_sz], _vp),
    "gpu_free": ([_vp], None),
    "gpu_memcpy_h2d": ([_vp, _vp, _sz], _i),
    "gpu_memcpy_d2h": ([_vp, _vp, _sz], _i),
    "gpu_memcpy_d2d": ([_vp, _vp, _sz], _i),
    "gpu_sync": ([], _i),
    "get_gpu_info": ([ctypes.c_char_p, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)], _i),
    "nvfp4_b200_abi_version": ([], _i),
    "launch_nvfp4_gemv": _GEMV_SIG,
    "launch_nvfp4_gemv_v8": _GEMV_SIG,
    "launch_nvfp4_gemv_v4": _GEMV_SIG,
    "launch_nvfp4_gemv_v5": _GEMV_SIG,
    "launch_nvfp4_gemv_v6": _GEMV_SIG,
    "launch_nvfp4_gemv_v7": _GEMV_SIG,
    "launch_nvfp4_gemvnl": _GEMV_SIG,
    "launch_nvfp4_gemv2": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _vp], _i),
    "launch_nvfp4_gemv2i": ([_vp, _vp, _vp, _vp, _i, _i, _vp], _i),
    "nvfp4_b200_gemv_config": ([_i, _i, _i], _i),
    "nvfp4_gemv_status": ([_i], _i),
    "nvfp4_b200_gemv_stream_config": ([_i, _i, _i, _i, _i, _i, _i], _i),
    "launch_nvfp4_gemmtc_v5": ([_vp, _vp, _vp, _vp, _i, _i, _i, _vp], _i),
    "launch_nvfp4_gemm_w4a16_ex": ([_vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _vp], _i),
    "get_kernel_shared_mem_bytes": ([], _i),
    "nvfp4_gemm_status": ([_i], _i),
    "launch_rmsnorm": ([_vp, _ll, _vp, _vp, _i, _i, _f, _vp], _i),
    "launch_rope_qk": ([_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp], _i),
    "launch_silu_mul": ([_vp, _vp, _vp, _i, _vp], _i),
    "launch_attn_decode": ([_vp] * 6 + [_i, _f, _vp], _i),
    "launch_attn_decode_heads": ([_vp] * 6 + [_i, _i, _i, _f, _vp], _i),
    "launch_nvfp4_gemv_fused": ([_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _f, _i, _vp, _vp], _i),
    "nvfp4_attn_split_scratch_bytes": ([_i], _ll),
    "launch_attn_decode_split": ([_vp] * 7 + [_i, _i, _i, _f, _vp], _i),
    "launch_embed_gather": ([_vp, _vp, _vp, _i, _ll, _vp], _i),
    "launch_attn_prep": ([_vp] * 10 + [_i, _i, _i, _f, _vp], _i),
    "launch_argmax_advance": ([_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp], _i),
    "launch_residual_add": ([_vp, _vp, _i, _vp], _i),
    "launch_argmax_slice": ([_vp, _i, _ll, _vp, _vp], _i),
    "launch_pick_global_argmax": ([_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp], _i),
    "nvfp4_comm_buffer_bytes": ([_i], _ll),
    "nvfp4_comm_data_offset": ([_i, _i], _ll),
    "nvfp4_comm_init": ([_vp, _i], _i),
    "nvfp4_ipc_get_handle": ([_vp, _vp], _i),
    "nvfp4_ipc_open_handle": ([_vp], _vp),
    "nvfp4_ipc_close_handle": ([_vp], _i),
    "nvfp4_comm_status": ([_vp], _i),
    "launch_nvfp4_gemv_allreduce": ([_vp, _vp, _vp, _vp, _i, _i, ctypes.POINTER(_vp), _i, _i, _i, _i,
                                     _vp], _i),
    "launch_allreduce_residual": ([_vp, ctypes.POINTER(_vp), _i, _i, _i, _i, _vp], _i),
    "launch_nvfp4_gemv_fused_ar": ([_vp, _vp, _vp, _vp, _i, _i, _vp, _f, _i, ctypes.POINTER(_vp), _i, _i,
                                    _i, _i, _vp, _i, _i, _vp], _i),
    "launch_argmax_exchange": ([_vp, _i, _ll, ctypes.POINTER(_vp), _i, _i, _i, _vp, _vp, _vp, _vp, _vp,
                                _vp, _i, _vp], _i),
    "launch_dn_fused": ([_vp] * 12 + [_f, _vp], _i),
    "launch_dn_fused_heads": ([_vp] * 12 + [_i, _i, _f, _vp], _i),
    "launch_transpose_f16": ([_vp, _ll, _vp, _ll, _i, _i, _vp], _i),
    "launch_add_transposed": ([_vp, _vp, _ll, _i, _i, _vp], _i),
    "launch_embed_rows": ([_vp, _vp, _vp, _i, _i, _ll, _vp], _i),
    "launch_silu_mul_rows": ([_vp, _vp, _i, _i, _vp], _i),
    "launch_attn_prep_tokens": ([_vp, _ll] + [_vp] * 4 + [_i, _i] + [_vp] * 4 + [_i, _i, _i, _f, _vp], _i),
    "launch_attn_prefill": ([_vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _f, _vp], _i),
    "nvfp4_dn_prefill_work_bytes": ([_i, _i, _i], _ll),
    "launch_dn_prefill": ([_vp, _ll] + [_vp] * 7 + [_ll, _vp, _i, _i, _i, _f, _vp], _i),
    "launch_nvfp4_decode_rows": ([_vp, _vp, _vp, _vp, _i, _i, _ll, _vp], _i),
    "launch_nvfp4_quant_dequant_T": ([_vp, _ll, _vp, _ll, _i, _i, _vp], _i),
    "launch_nvfp4_gemm_w4a4": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp], _i),
    "launch_nvfp4_encode": ([_vp, _vp, _vp, _i, _i, _vp], _i),
    "launch_nvfp4_gemm_fp4": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp], _i),
    "nvfp4_gemm_fp4_status": ([_i], _i),
    "nvfp4_b200_gemm_fp4_config": ([_i], None),
    "launch_nvfp4_gemv_tc": ([_vp, _vp, _vp, _vp, _i, _i, _vp], _i),
    "nvfp4_gemv_tc_status": ([_i], _i),
    "nvfp4_b200_gemv_tc_config": ([_i], None),
    "nvfp4_b200_gemm_config": ([_i], None),
    "nvfp4_b200_gemv_tc_ring": ([_i], None),
    "nvfp4_b200_gemv_tc_ctas": ([_i], None),
    "nvfp4_b200_gemv_tc_prefetch": ([_i], None),
    "launch_nvfp4_gemv_tc_fused": ([_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _f, _i, _vp, _vp], _i),
    "launch_nvfp4_mlp_tc": ([_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _vp], _i),
    "nvfp4_gemv_tc_wanted": ([_i, _i], _i),
    "nvfp4_gemv_tc_wanted_plain": ([_i, _i], _i),
    "nvfp4_b200_gemv_tc_config_plain": ([_i], None),
    "nvfp4_gemv_tc_prepare": ([], _i),
    "nvfp4_gemv_tc_probe": ([_vp], None),
    "launch_dn_fused_noalloc": ([_vp] * 11 + [_i, _i, _f, _vp], _i),
}

_LIB = None


def load(path: str | None = None) -> ctypes.CDLL:
    """Load the library once and attach argtypes/restype to every declared symbol."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(
            f"{p} is missing: build it with `python -m nvfp4_v100_b200.build` "
            "(needs nvcc; there is no CPU fallback)")
    lib = ctypes.CDLL(p)
    for name, (argtypes, restype) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise RuntimeError(f"{p} does not export `{name}`") from e
        fn.argtypes = argtypes
        fn.restype = restype
    if path is None:
        _LIB = lib
    return lib

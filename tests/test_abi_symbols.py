"""The shared library loads without a GPU and exports every symbol the header declares;
host-side argument validation returns the reference's error codes before any launch."""
import ctypes
import os
import re

from conftest import ROOT


def declared_functions():
    src = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", src)))


def test_header_symbols_exported(lib):
    names = declared_functions()
    assert "launch_nvfp4_gemv_v8" in names and "launch_dn_fused" in names and len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"missing export {n}"


def test_binding_table_matches_header():
    from nvfp4_v100_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_functions()


def declared_argument_counts():
    """name -> number of parameters, parsed from the header's declarations."""
    src = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    out = {}
    for name, args in re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(([^;{]*)\)\s*;", src):
        args = " ".join(args.split())
        out[name] = 0 if args in ("", "void") else args.count(",") + 1
    return out


def test_binding_argument_counts_match_header():
    # every .cu file is compiled against the header, so header == definitions; this closes the
    # remaining gap between the header and the ctypes table
    from nvfp4_v100_b200 import _lib

    counts = declared_argument_counts()
    for name, (argtypes, _res) in _lib.SIGNATURES.items():
        assert counts[name] == len(argtypes), (name, counts[name], len(argtypes))


def test_every_kernel_source_is_compiled_against_the_header():
    csrc = os.path.join(ROOT, "nvfp4_v100_b200", "csrc")
    assert '#include "nvfp4_b200.h"' in open(os.path.join(csrc, "common.cuh")).read()
    for f in os.listdir(csrc):
        if f.endswith(".cu"):
            assert '#include "common.cuh"' in open(os.path.join(csrc, f)).read(), f


def test_dll_aliases_resolve(lib):
    from nvfp4_v100_b200 import _lib, build

    for name in build.DLL_ALIASES:
        p = os.path.join(_lib.KDIR, name)
        assert os.path.exists(p), p
        h = ctypes.CDLL(p)
        assert hasattr(h, "gpu_malloc")


def test_gemv_argument_validation_is_host_side(lib):
    # K not a multiple of 32 -> -2 (reference: kernels/nvfp4_gemv.cu:842), checked before launch
    one = ctypes.c_void_p(0x1000)
    for fn in (lib.launch_nvfp4_gemv, lib.launch_nvfp4_gemv_v8, lib.launch_nvfp4_gemvnl):
        assert fn(one, one, one, one, 16, 48, None) == -2
        assert fn(one, one, one, one, 16, 0, None) == -2
        assert fn(one, one, one, one, 0, 64, None) == -2
        assert fn(None, one, one, one, 16, 64, None) == -2
        assert fn(ctypes.c_void_p(0x1008), one, one, one, 16, 64, None) == -2  # misaligned weights
    assert lib.launch_nvfp4_gemv_v7(one, one, one, one, 16, 96, None) == -2     # v7: K % 64
    assert lib.launch_nvfp4_gemv2(one, one, one, None, one, 16, 64, None) == -2


def test_fused_op_argument_validation(lib):
    one = ctypes.c_void_p(0x1000)
    assert lib.launch_rmsnorm(one, 8, one, one, 0, 8, 1e-6, None) == -1
    assert lib.launch_rmsnorm(one, 8, one, one, 1, 0, 1e-6, None) == -1
    assert lib.launch_rope_qk(one, one, one, one, one, one, 0, 0, None) == -1
    assert lib.launch_silu_mul(one, one, one, 0, None) == -1
    assert lib.launch_attn_decode(one, one, one, one, one, one, 0, 1.0, None) == -2
    assert lib.launch_attn_decode(one, one, one, one, one, one, 1 << 20, 1.0, None) == -2
    args = [one] * 12
    args[3] = None
    assert lib.launch_dn_fused(*args, 1e-6, None) == -1
    assert lib.nvfp4_b200_gemv_config(3, 0, 0) == -2
    assert lib.nvfp4_b200_gemv_config(0, 0, 0) == 0

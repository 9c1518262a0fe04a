"""Cross-check on the GPU against the reference's own CUDA kernels, recompiled unchanged for
sm_100a by oracle/Makefile into oracle/_ref/ (git-ignored; built where the reference tree is
mounted and shipped to the GPU box as binaries).  Skipped when those binaries are absent.

What is asserted:
  * RoPE, silu*mul: bit-identical (same formula, same rounding points, no reductions);
  * RMSNorm, attention decode, DeltaNet step: within one fp16 step (our reductions are shuffle
    trees, the reference's are thread-serial loops), fp32 state within 1e-5;
  * GEMV: both kernels against the float64 truth; ours (fp32 accumulation of exact products) must
    be at least as accurate as the reference's fp16 multiply chain.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import ROOT
from oracle import nvfp4_codec_oracle as oc
from tests.gpu_util import dev, ptr, stream, ulp_diff_f16
from tests.test_fused_gpu import make_dn_inputs

pytestmark = pytest.mark.gpu
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
vp = ctypes.c_void_p


def ref_lib(name):
    p = os.path.join(REF_DIR, f"ref_{name}.so")
    if not os.path.exists(p):
        pytest.skip(f"{p} not built (needs the reference tree: make -C oracle)")
    return ctypes.CDLL(p)


def test_rope_and_silu_bit_identical(lib):
    ref = ref_lib("nvfp4_rope_silu")
    rng = np.random.default_rng(0)
    q, k = dev(rng.standard_normal((24, 256)).astype(np.float16)), dev(rng.standard_normal((4, 256)).astype(np.float16))
    ang = rng.uniform(0, 6.28, 256)
    c, s = dev(np.cos(ang).astype(np.float16)), dev(np.sin(ang).astype(np.float16))
    outs = []
    for L in (lib, ref):
        qo, ko = torch.zeros_like(q), torch.zeros_like(k)
        assert L.launch_rope_qk(ptr(q), ptr(k), ptr(c), ptr(s), ptr(qo), ptr(ko), 24, 4, stream()) == 0
        torch.cuda.synchronize()
        outs.append((qo.cpu().numpy(), ko.cpu().numpy()))
    assert np.array_equal(outs[0][0].view(np.uint16), outs[1][0].view(np.uint16))
    assert np.array_equal(outs[0][1].view(np.uint16), outs[1][1].view(np.uint16))

    bits = np.arange(0x10000, dtype=np.uint32).astype(np.uint16).view(np.float16)
    g = bits[np.isfinite(bits)]
    u = rng.standard_normal(len(g)).astype(np.float16)
    dg, du = dev(g), dev(u)
    res = []
    for L in (lib, ref):
        o = torch.zeros(len(g), dtype=torch.float16, device="cuda")
        assert L.launch_silu_mul(ptr(dg), ptr(du), ptr(o), len(g), stream()) == 0
        torch.cuda.synchronize()
        res.append(o.cpu().numpy())
    assert np.array_equal(res[0].view(np.uint16), res[1].view(np.uint16))


def test_rmsnorm_vs_reference_kernel(lib):
    ref = ref_lib("nvfp4_rmsnorm")
    rng = np.random.default_rng(1)
    for rows, n, stride in ((1, 5120, 5120), (24, 256, 512), (4, 256, 256)):
        x = dev(rng.standard_normal(rows * stride).astype(np.float16))
        w1 = dev((1 + 0.1 * rng.standard_normal(n)).astype(np.float32))
        res = []
        for L in (lib, ref):
            L.launch_rmsnorm.argtypes = [vp, ctypes.c_longlong, vp, vp, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_float, vp]
            o = torch.zeros(rows * n, dtype=torch.float16, device="cuda")
            assert L.launch_rmsnorm(ptr(x), stride, ptr(w1), ptr(o), rows, n, 1e-6, stream()) == 0
            torch.cuda.synchronize()
            res.append(o.cpu().numpy())
        d = ulp_diff_f16(res[0], res[1])
        assert d.max() <= 1 and (d == 0).mean() > 0.99, (d.max(), (d == 0).mean())


@pytest.mark.parametrize("name,max_len,L", [("nvfp4_attn_decode", 3072, 575),
                                            ("nvfp4_attn_decode", 3072, 3072),
                                            ("nvfp4_attn_decode_1024", 1024, 1),
                                            ("nvfp4_attn_decode_1024", 1024, 600)])
def test_attn_decode_vs_reference_kernel(lib, name, max_len, L):
    ref = ref_lib(name)
    rng = np.random.default_rng(L)
    q = dev(rng.standard_normal((24, 256)).astype(np.float16))
    gate = dev(rng.standard_normal((24, 256)).astype(np.float16))
    keys = dev(rng.standard_normal((4, max_len, 256)).astype(np.float16))
    vals = dev(rng.standard_normal((4, max_len, 256)).astype(np.float16))
    cum = torch.tensor([L], dtype=torch.int64, device="cuda")
    res = []
    for Lb in (lib, ref):
        Lb.launch_attn_decode.argtypes = [vp] * 6 + [ctypes.c_int, ctypes.c_float, vp]
        o = torch.zeros(24 * 256, dtype=torch.float16, device="cuda")
        rc = Lb.launch_attn_decode(ptr(q), ptr(keys), ptr(vals), ptr(cum), ptr(gate), ptr(o),
                                   max_len, 256 ** -0.5, stream())
        torch.cuda.synchronize()
        assert rc == 0
        res.append(o.cpu().numpy())
    d = ulp_diff_f16(res[0], res[1])
    assert d.max() <= 2 and (d == 0).mean() > 0.98, (d.max(), (d == 0).mean())


def test_dn_fused_vs_reference_kernel(lib):
    ref = ref_lib("nvfp4_dn_fused")
    x = make_dn_inputs(3)
    res = []
    for Lb in (lib, ref):
        Lb.launch_dn_fused.argtypes = [vp] * 12 + [ctypes.c_float, vp]
        d = {k: dev(v) for k, v in x.items()}
        scratch = torch.zeros(10240, dtype=torch.float32, device="cuda")
        out = torch.zeros(6144, dtype=torch.float16, device="cuda")
        for step in range(3):
            rc = Lb.launch_dn_fused(ptr(d["mixed"]), ptr(d["z"]), ptr(d["b"]), ptr(d["a"]),
                                    ptr(d["conv_w"]), ptr(d["conv_state"]), ptr(d["A_log"]),
                                    ptr(d["dt_bias"]), ptr(d["norm_w"]), ptr(d["state"]),
                                    ptr(scratch), ptr(out), 1e-6, stream())
            assert rc == 0
        torch.cuda.synchronize()
        res.append((out.cpu().numpy(), d["state"].cpu().numpy(), d["conv_state"].cpu().numpy(),
                    scratch.cpu().numpy()))
    assert np.array_equal(res[0][2].view(np.uint16), res[1][2].view(np.uint16))   # conv state
    assert np.array_equal(res[0][3], res[1][3])                                   # conv + silu
    assert np.abs(res[0][1] - res[1][1]).max() <= 1e-5 * np.abs(res[1][1]).max()
    # the output passes through four fp16 roundings in a row (o, xn, xn*w, *silu(z)); after three
    # steps with independently evolving fp32 state a few elements sit on opposite sides of a
    # rounding boundary at more than one of them
    d = ulp_diff_f16(res[0][0], res[1][0])
    assert d.max() <= 8 and (d == 0).mean() > 0.95, (d.max(), (d == 0).mean())


def test_gemv_accuracy_vs_reference_kernel(lib):
    ref = ref_lib("nvfp4_gemv")
    M, K = 5120, 5120
    w = oc.synthetic_weight(M, K, seed=0)
    p, s = oc.encode(w)
    a = oc.synthetic_act(K, seed=0)
    truth = oc.gemv_f64(p, s, a)
    dp, ds, da = dev(p), dev(s), dev(a)
    errs = []
    for Lb in (lib, ref):
        Lb.launch_nvfp4_gemv_v8.argtypes = [vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, vp]
        o = torch.zeros(M, dtype=torch.float16, device="cuda")
        assert Lb.launch_nvfp4_gemv_v8(ptr(dp), ptr(ds), ptr(da), ptr(o), M, K, stream()) == 0
        torch.cuda.synchronize()
        errs.append(oc.rel_error_floored(o.cpu().numpy(), truth))
    ours, theirs = errs
    print(f"\nGEMV 5120x5120 max floored rel err: ours {ours.max():.2e}, reference v8 kernel "
          f"{theirs.max():.2e}; mean ours {ours.mean():.2e}, reference {theirs.mean():.2e}")
    assert ours.max() <= 1e-3
    assert ours.mean() <= theirs.mean()

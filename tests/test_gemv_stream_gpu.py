"""The ring-streaming GEMV kernel (TMA tensor copies into a shared-memory ring) against the
CPU oracle and against the register-streaming kernel, through the C ABI.

Tolerance as in test_gemv_gpu.py: max |y - ref| / max(|ref|, 1e-3 max|ref|) <= 1e-3 against the
float64 product of the exactly decoded matrix.  The two kernels add the same exact products in a
different order, so they agree to within that bound (not bit for bit).
"""
import ctypes

import numpy as np
import pytest
import torch

from nvfp4_v100_b200.engine import interleave_gate_up
from oracle import fused_ops_oracle as fo
from oracle import nvfp4_codec_oracle as oc
from tests.gpu_util import dev, gemv, ptr, stream, ulp_diff_f16

pytestmark = pytest.mark.gpu
TOL = 1e-3


def stream_cfg(lib, warps=0, smem_kb=0, stage_kb=0, min_stages=0, ctas=0, rb=0, on=1):
    """Switch the ring kernel on (it is off by default) with the given tuning values."""
    assert lib.nvfp4_b200_gemv_stream_config(warps, smem_kb, stage_kb, min_stages, ctas, rb, on) == 0


@pytest.fixture(autouse=True)
def _reset(lib):
    lib.nvfp4_gemv_status(1)
    stream_cfg(lib)
    yield
    stream_cfg(lib, on=0)
    assert lib.nvfp4_gemv_status(0) == 0, "a bounded wait inside the ring GEMV ran out"


def check(y, p, s, a):
    ref = oc.gemv_f64(p, s, a)
    rel = oc.rel_error_floored(y, ref)
    assert np.isfinite(y.astype(np.float64)).all()
    assert rel.max() <= TOL, f"max rel {rel.max():.3e}"
    assert (y == ref.astype(np.float16)).mean() > 0.95


# rows that do not fill a 16-row tile, rows that do not divide over the SMs, one to many K chunks
SHAPES = [(1, 256), (7, 512), (16, 256), (17, 1024), (48, 5120), (100, 768), (147, 2560),
          (149, 256), (1024, 5120), (33, 17408), (5120, 5120), (257, 6144), (5120, 17408),
          (2368, 5120), (4737, 1280)]


@pytest.mark.parametrize("M,K", SHAPES)
def test_ring_kernel_against_oracle(lib, M, K):
    w = oc.synthetic_weight(M, K, seed=M * 31 + K)
    p, s = oc.encode(w)
    a = oc.synthetic_act(K, seed=K)
    rc, y = gemv(lib, p, s, a)
    assert rc == 0
    check(y, p, s, a)
    stream_cfg(lib, on=0)                            # the register-streaming kernel
    rc, y_old = gemv(lib, p, s, a)
    assert rc == 0
    assert oc.rel_error_floored(y, y_old.astype(np.float64)).max() <= TOL


@pytest.mark.parametrize("cfg", [
    dict(warps=4), dict(warps=8), dict(warps=12), dict(rb=16), dict(warps=12, rb=16, stage_kb=5),
    dict(smem_kb=100, warps=4), dict(stage_kb=18, warps=4), dict(stage_kb=5), dict(stage_kb=5, min_stages=2),
    dict(stage_kb=14, warps=4, min_stages=3), dict(ctas=2, warps=4), dict(min_stages=2),
])
def test_ring_kernel_configurations(lib, cfg):
    # one to 24 K chunks per row tile, ragged last chunks (zero-filled by the tensor map), ragged
    # last row tiles (boxes of four rows), two to four stages per warp, every warp count
    for M, K in ((200, 1024), (531, 5120), (70, 17408), (3000, 6144)):
        w = oc.synthetic_weight(M, K, seed=M + K)
        p, s = oc.encode(w)
        a = oc.synthetic_act(K, seed=K + 3)
        stream_cfg(lib, **cfg)
        rc, y = gemv(lib, p, s, a)
        assert rc == 0
        check(y, p, s, a)


def test_ring_kernel_repeated_launches_and_scale_extremes(lib):
    # back-to-back dependent launches (programmatic dependent launch: the next kernel's ring is
    # filled while this one runs) writing and re-reading the same buffers
    M = K = 1024
    w = oc.synthetic_weight(M, K, seed=5, sigma=0.03)
    p, s = oc.encode(w)
    x0 = oc.synthetic_act(K, seed=6)
    d_p, d_s = dev(p), dev(s)
    bufs = [dev(x0), torch.zeros(M, dtype=torch.float16, device="cuda")]
    want = x0
    for i in range(6):
        rc = lib.launch_nvfp4_gemv_v8(ptr(d_p), ptr(d_s), ptr(bufs[i & 1]), ptr(bufs[(i + 1) & 1]),
                                      M, K, stream())
        assert rc == 0
        want = oc.gemv_f64(p, s, want).astype(np.float16)
    torch.cuda.synchronize()
    got = bufs[0].cpu().numpy()
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert err.max() <= 2e-2 * np.abs(want.astype(np.float64)).max()   # six chained roundings
    # scale byte 0 -> +0, byte 254 -> inf, as the reference kernels decode them
    pk = np.full((32, 128), 0x22, dtype=np.uint8)
    sc = np.full((32, 16), 127, dtype=np.uint8)
    sc[1, :] = 0
    sc[18, :] = 254
    rc, y = gemv(lib, pk, sc, np.ones(256, dtype=np.float16))
    assert rc == 0
    assert y[0] == 256 and y[1] == 0 and np.isinf(y[18]) and y[31] == 256


def fused(lib, p, s, x, M, K, pro_w1=None, epi=0, residual=None, out_rows=None):
    d_p, d_s, d_x = dev(p), dev(s), dev(x.astype(np.float16))
    n = out_rows or M
    out = torch.full((n + 8,), float("nan"), dtype=torch.float16, device="cuda")
    d_w = dev(pro_w1) if pro_w1 is not None else None
    d_r = dev(residual.astype(np.float16)) if residual is not None else None
    z = ctypes.c_void_p(0)
    rc = lib.launch_nvfp4_gemv_fused(ptr(d_p), ptr(d_s), ptr(d_x), ptr(out), M, K,
                                     0 if d_w is None else 1, z if d_w is None else ptr(d_w), 1e-6,
                                     epi, z if d_r is None else ptr(d_r), stream())
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.isnan(o[n:]).all()
    return rc, o[:n]


@pytest.mark.parametrize("warps,stage_kb", [(4, 0), (8, 0), (12, 5)])
@pytest.mark.parametrize("M,K", [(772, 256), (5120, 5120), (1000, 512), (40, 6144)])
def test_ring_fused_rmsnorm_and_residual(lib, M, K, warps, stage_kb):
    w = oc.synthetic_weight(M, K, seed=M + K)
    p, s = oc.encode(w)
    x = oc.synthetic_act(K, seed=3)
    w1 = (1 + 0.1 * np.random.default_rng(1).standard_normal(K)).astype(np.float32)
    res = np.random.default_rng(2).standard_normal(M).astype(np.float16)
    xn = fo.rmsnorm(x[None], w1, 1e-6)[0]
    y = oc.gemv_f64(p, s, xn).astype(np.float16)
    want = (res.astype(np.float64) + y.astype(np.float64)).astype(np.float16)
    stream_cfg(lib, warps=warps, stage_kb=stage_kb)
    rc, got = fused(lib, p, s, x, M, K, pro_w1=w1, epi=1, residual=res)
    assert rc == 0
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert err.max() <= 2e-3 * max(1.0, np.abs(want.astype(np.float64)).max())
    assert (ulp_diff_f16(got, want) <= 1).mean() > 0.98
    # same call on the register-streaming kernel
    stream_cfg(lib, on=0)
    rc, old = fused(lib, p, s, x, M, K, pro_w1=w1, epi=1, residual=res)
    assert rc == 0
    assert (ulp_diff_f16(got, old) <= 1).mean() > 0.98


@pytest.mark.parametrize("inter,K", [(512, 256), (17408, 5120), (48, 1024)])
def test_ring_fused_silu_mul(lib, inter, K):
    g_w = oc.synthetic_weight(inter, K, seed=inter, sigma=0.05)
    u_w = oc.synthetic_weight(inter, K, seed=inter + 1, sigma=0.05)
    gp, gs = oc.encode(g_w)
    upk, us = oc.encode(u_w)
    x = oc.synthetic_act(K, seed=4)
    g = oc.gemv_f64(gp, gs, x).astype(np.float16)
    u = oc.gemv_f64(upk, us, x).astype(np.float16)
    want = fo.silu_mul(g, u)
    p = interleave_gate_up(torch.from_numpy(gp), torch.from_numpy(upk)).numpy()
    s = interleave_gate_up(torch.from_numpy(gs), torch.from_numpy(us)).numpy()
    w1 = np.ones(K, dtype=np.float32)
    for pro in (None, w1):
        xin = x
        rc, got = fused(lib, p, s, xin, 2 * inter, K, pro_w1=pro, epi=2, out_rows=inter)
        assert rc == 0
        if pro is not None:      # normalised input: compare with the oracle on the same input
            xn = fo.rmsnorm(x[None], w1, 1e-6)[0]
            gg = oc.gemv_f64(gp, gs, xn).astype(np.float16)
            uu = oc.gemv_f64(upk, us, xn).astype(np.float16)
            ref = fo.silu_mul(gg, uu)
        else:
            ref = want
        d = ulp_diff_f16(got, ref)
        assert (d == 0).mean() > 0.98, (d == 0).mean()
        err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
        assert (err <= 4e-3 * np.abs(ref.astype(np.float64)) + 1e-6).all(), d.max()


def test_linearity_full_size_on_the_ring_kernel(lib):
    # W(a+b) = Wa + Wb exactly when every operand is a small integer (all sums exact in fp32)
    M, K = 5120, 17408
    rng = np.random.default_rng(1)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = np.full((M, K // 16), 127 - 4, dtype=np.uint8)
    a = rng.integers(-2, 3, size=K).astype(np.float16)
    b = rng.integers(-2, 3, size=K).astype(np.float16)
    for v in (a, b, a + b):
        _, y = gemv(lib, p, s, v)
        ref = oc.gemv_f64(p, s, v)
        assert np.array_equal(y.astype(np.float64), ref.astype(np.float16).astype(np.float64))

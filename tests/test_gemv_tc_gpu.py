"""GEMV on the FP4 tensor-core path (launch_nvfp4_gemv_tc) against the CPU oracle.

Oracle and tolerance as for the register-streaming GEMV: codec decode of the weight bytes, float64
dot product with the fp16 activation (kernels/nvfp4_gemv.cu:38-69 semantics); max |y - ref| /
max(|ref|, 1e-3 max|ref|) <= 1e-3.  The activation enters the tensor core as exact base-4 digits,
so inputs that stress the digit expansion are covered: zero blocks, a 2^20 spread inside one
block, fp16 subnormals, the largest fp16 values."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_codec_oracle as oc
from tests.gpu_util import dev, ptr, stream

pytestmark = pytest.mark.gpu


def run(lib, p, s, x):
    M, K = p.shape[0], p.shape[1] * 2
    d_p, d_s, d_x = dev(p), dev(s), dev(x)
    out = torch.full((M + 16,), float("nan"), dtype=torch.float16, device="cuda")
    lib.nvfp4_gemv_tc_status(1)
    rc = lib.launch_nvfp4_gemv_tc(ptr(d_p), ptr(d_s), ptr(d_x), ptr(out), M, K, stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert lib.nvfp4_gemv_tc_status(0) == 0, "a bounded wait inside the kernel ran out"
    o = out.cpu().numpy()
    assert np.isnan(o[M:]).all(), "wrote past the output"
    return o[:M]


def check(y, p, s, x, tol=1e-3):
    ref = oc.decode_f64(p, s) @ x.astype(np.float64)
    assert np.isfinite(y.astype(np.float64)).all()
    rel = oc.rel_error_floored(y, ref)
    assert rel.max() <= tol, (rel.max(), int(rel.argmax()))


@pytest.mark.parametrize("M,K", [
    (128, 256), (1, 256), (300, 512), (129, 1024), (1024, 5120), (5120, 5120), (33, 17408),
    (6144, 5120), (17408, 5120), (5120, 17408), (40000, 1024), (5120, 6144), (48, 5120),
])
def test_against_oracle(lib, M, K):
    w = oc.synthetic_weight(M, K, seed=M + K)
    p, s = oc.encode(w)
    x = oc.synthetic_act(K, seed=K)
    check(run(lib, p, s, x), p, s, x)


def test_activation_extremes(lib):
    M, K = 384, 1024
    rng = np.random.default_rng(3)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
    x = rng.standard_normal(K).astype(np.float16)
    x[:32] = 0                                  # two all-zero blocks
    x[32] = 1024.0; x[33] = 2.0 ** -10          # a 2^20 spread inside one block
    x[48:64] = np.float16(6e-8) * rng.integers(-9, 10, 16).astype(np.float16)   # subnormals
    x[64] = 60000.0; x[65] = -60000.0; x[66] = 30000.0   # near the fp16 maximum
    x[80:96] = -x[80:96]
    y = run(lib, p, s, x)
    check(y, p, s, x)
    # exactness of the digit expansion: scaling x by a power of two scales y exactly (no block
    # changes its digits), as long as nothing leaves the fp16 range
    x2 = (x.astype(np.float32) * 0.25).astype(np.float16)
    keep = (x2.astype(np.float32) * 4 == x.astype(np.float32))
    x, x2 = np.where(keep, x, 0).astype(np.float16), np.where(keep, x2, 0).astype(np.float16)
    ya, yb = run(lib, p, s, x).astype(np.float32), run(lib, p, s, x2).astype(np.float32)
    normal = np.abs(yb) >= 2.0 ** -13
    assert np.array_equal(ya[normal], 4 * yb[normal])


def test_repeated_launches_are_identical_and_leave_the_workspace_clean(lib):
    M, K = 5120, 5120
    p, s = oc.encode(oc.synthetic_weight(M, K, seed=1))
    x = oc.synthetic_act(K, seed=2)
    y0 = run(lib, p, s, x)
    for _ in range(3):
        assert np.array_equal(run(lib, p, s, x), y0)
    # another shape in between uses the same counters and slots
    p2, s2 = oc.encode(oc.synthetic_weight(300, 2048, seed=4))
    x2 = oc.synthetic_act(2048, seed=5)
    check(run(lib, p2, s2, x2), p2, s2, x2)
    assert np.array_equal(run(lib, p, s, x), y0)


def fused(lib, p, s, x, M, K, pro_w1=None, epi=0, residual=None, out_rows=None, entry=None):
    import ctypes

    d_p, d_s, d_x = dev(p), dev(s), dev(x.astype(np.float16))
    n = out_rows or M
    out = torch.full((n + 8,), float("nan"), dtype=torch.float16, device="cuda")
    d_w = dev(pro_w1) if pro_w1 is not None else None
    d_r = dev(residual.astype(np.float16)) if residual is not None else None
    z = ctypes.c_void_p(0)
    lib.nvfp4_gemv_tc_status(1)
    rc = (entry or lib.launch_nvfp4_gemv_tc_fused)(
        ptr(d_p), ptr(d_s), ptr(d_x), ptr(out), M, K, 0 if d_w is None else 1,
        z if d_w is None else ptr(d_w), 1e-6, epi, z if d_r is None else ptr(d_r), stream())
    torch.cuda.synchronize()
    assert rc == 0 and lib.nvfp4_gemv_tc_status(0) == 0
    o = out.cpu().numpy()
    assert np.isnan(o[n:]).all()
    return o[:n]


@pytest.mark.parametrize("M,K", [(772, 256), (5120, 5120), (100, 10240), (1000, 512), (5120, 17408)])
def test_fused_rmsnorm_prologue_and_residual(lib, M, K):
    from oracle import fused_ops_oracle as fo

    p, s = oc.encode(oc.synthetic_weight(M, K, seed=M + K))
    x = oc.synthetic_act(K, seed=3)
    res = np.random.default_rng(2).standard_normal(M).astype(np.float16)
    if K <= 10240:
        w1 = (1 + 0.1 * np.random.default_rng(1).standard_normal(K)).astype(np.float32)
        xn = fo.rmsnorm(x[None], w1, 1e-6)[0]
    else:
        w1, xn = None, x          # the prologue takes K <= 11520; the residual epilogue any K
    y = oc.gemv_f64(p, s, xn).astype(np.float16)
    want = (res.astype(np.float64) + y.astype(np.float64)).astype(np.float16)
    got = fused(lib, p, s, x, M, K, pro_w1=w1, epi=1, residual=res)
    # the normalised activation may differ from the oracle's in a few last bits, which moves y by
    # at most ~1e-3 of its scale; against the residual sum that is a couple of fp16 steps
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert err.max() <= 2e-3 * max(1.0, np.abs(y.astype(np.float64)).max())


@pytest.mark.parametrize("inter,K", [(512, 256), (17408, 5120), (40, 1024)])
def test_fused_silu_mul_epilogue(lib, inter, K):
    from nvfp4_v100_b200.engine import interleave_gate_up
    from oracle import fused_ops_oracle as fo
    from tests.gpu_util import ulp_diff_f16

    gp, gs = oc.encode(oc.synthetic_weight(inter, K, seed=inter, sigma=0.05))
    upk, us = oc.encode(oc.synthetic_weight(inter, K, seed=inter + 1, sigma=0.05))
    x = oc.synthetic_act(K, seed=4)
    w1 = (1 + 0.1 * np.random.default_rng(5).standard_normal(K)).astype(np.float32)
    xn = fo.rmsnorm(x[None], w1, 1e-6)[0]
    want = fo.silu_mul(oc.gemv_f64(gp, gs, xn).astype(np.float16), oc.gemv_f64(upk, us, xn).astype(np.float16))
    p = interleave_gate_up(torch.from_numpy(gp), torch.from_numpy(upk)).numpy()
    s = interleave_gate_up(torch.from_numpy(gs), torch.from_numpy(us)).numpy()
    got = fused(lib, p, s, x, 2 * inter, K, pro_w1=w1, epi=2, out_rows=inter)
    d = ulp_diff_f16(got, want)
    assert (d == 0).mean() > 0.97, (d == 0).mean()
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert (err <= 6e-3 * np.abs(want.astype(np.float64)) + 2e-6).all(), d.max()
    # the routed entry (launch_nvfp4_gemv_fused sends this size to the tensor-core kernel when the
    # matrix is large enough) gives the same bits as the direct one
    if lib.nvfp4_gemv_tc_wanted(2 * inter, K):
        again = fused(lib, p, s, x, 2 * inter, K, pro_w1=w1, epi=2, out_rows=inter,
                      entry=lib.launch_nvfp4_gemv_fused)
        assert np.array_equal(again, got)


def test_routing_rule(lib):
    assert lib.nvfp4_gemv_tc_prepare() == 0
    assert lib.nvfp4_gemv_tc_wanted(34816, 5120) == 1 and lib.nvfp4_gemv_tc_wanted(5120, 5120) == 0
    lib.nvfp4_b200_gemv_tc_config(0)
    assert lib.nvfp4_gemv_tc_wanted(34816, 5120) == 0
    lib.nvfp4_b200_gemv_tc_config(35)
    assert lib.nvfp4_gemv_tc_wanted(34816, 5120) == 1 and lib.nvfp4_gemv_tc_wanted(34816, 5100) == 0


def test_argument_validation(lib):
    import ctypes

    one = ctypes.c_void_p(0x1000)
    assert lib.launch_nvfp4_gemv_tc(one, one, one, one, 16, 384, None) == -2     # K % 256
    assert lib.launch_nvfp4_gemv_tc(one, one, one, one, 0, 1024, None) == -2
    assert lib.launch_nvfp4_gemv_tc(None, one, one, one, 16, 1024, None) == -2
    assert lib.launch_nvfp4_gemv_tc(ctypes.c_void_p(0x1008), one, one, one, 16, 1024, None) == -2


@pytest.mark.parametrize("hidden,inter", [(256, 512), (1024, 2816), (5120, 17408)])
def test_mlp_block_in_one_launch(lib, hidden, inter):
    # launch_nvfp4_mlp_tc = [RMSNorm -> gate/up GEMV -> silu*mul] and [down GEMV -> residual add] in
    # one kernel with a grid-wide barrier between the phases.  Checked against the two fused
    # launches it replaces (same arithmetic; bit-identical when both use the same grid, i.e. at
    # full size) and against the float64 oracle of the chain.
    import ctypes

    from nvfp4_v100_b200.engine import interleave_gate_up
    from oracle import fused_ops_oracle as fo

    rng = np.random.default_rng(hidden + inter)
    gp, gs = oc.encode(oc.synthetic_weight(inter, hidden, seed=1, sigma=0.05))
    upk, us = oc.encode(oc.synthetic_weight(inter, hidden, seed=2, sigma=0.05))
    dp, ds = oc.encode(oc.synthetic_weight(hidden, inter, seed=3, sigma=0.02))
    h0 = rng.standard_normal(hidden).astype(np.float16)
    w1 = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    p = interleave_gate_up(torch.from_numpy(gp), torch.from_numpy(upk)).numpy()
    s = interleave_gate_up(torch.from_numpy(gs), torch.from_numpy(us)).numpy()
    d_p, d_s, d_dp, d_ds, d_w = dev(p), dev(s), dev(dp), dev(ds), dev(w1)
    z = ctypes.c_void_p(0)

    # the two launches
    h_a = dev(h0.copy())
    act_a = torch.zeros(inter, dtype=torch.float16, device="cuda")
    assert lib.launch_nvfp4_gemv_tc_fused(ptr(d_p), ptr(d_s), ptr(h_a), ptr(act_a), 2 * inter, hidden, 1,
                                          ptr(d_w), 1e-6, 2, z, stream()) == 0
    assert lib.launch_nvfp4_gemv_tc_fused(ptr(d_dp), ptr(d_ds), ptr(act_a), ptr(h_a), hidden, inter, 0,
                                          z, 1e-6, 1, ptr(h_a), stream()) == 0
    # the one launch, three times in a row (the barrier and the slots must reset themselves)
    lib.nvfp4_gemv_tc_status(1)
    outs = []
    for _ in range(3):
        h_b = dev(h0.copy())
        act_b = torch.full((inter + 8,), float("nan"), dtype=torch.float16, device="cuda")
        rc = lib.launch_nvfp4_mlp_tc(ptr(d_p), ptr(d_s), ptr(d_dp), ptr(d_ds), ptr(h_b), ptr(act_b),
                                     ptr(d_w), 1e-6, inter, hidden, stream())
        torch.cuda.synchronize()
        assert rc == 0 and lib.nvfp4_gemv_tc_status(0) == 0
        assert bool(torch.isnan(act_b[inter:]).all())
        outs.append((h_b.cpu().numpy(), act_b[:inter].cpu().numpy()))
    torch.cuda.synchronize()
    for hb, ab in outs[1:]:
        assert np.array_equal(hb, outs[0][0]) and np.array_equal(ab, outs[0][1])
    ha, aa = h_a.cpu().numpy(), act_a.cpu().numpy()
    hb, ab = outs[0]
    if hidden == 5120:
        # same grid in both forms: the same bits (the two fused launches are checked against the
        # oracle at this size in test_fused_silu_mul_epilogue / test_fused_rmsnorm_prologue_and_residual)
        assert np.array_equal(ab, aa) and np.array_equal(hb, ha)
        return
    # smaller grids differ between the forms (fp32 partial sums are grouped differently): oracle
    xn = fo.rmsnorm(h0[None], w1, 1e-6)[0]
    act_ref = fo.silu_mul(oc.gemv_f64(gp, gs, xn).astype(np.float16), oc.gemv_f64(upk, us, xn).astype(np.float16))
    err = np.abs(ab.astype(np.float64) - act_ref.astype(np.float64))
    assert (err <= 2e-2 * np.abs(act_ref.astype(np.float64)) + 1e-4 * np.abs(act_ref).max()).all()
    y = oc.gemv_f64(dp, ds, ab)                  # the down projection of the act the kernel produced
    want = h0.astype(np.float64) + y.astype(np.float16).astype(np.float64)
    assert np.abs(hb.astype(np.float64) - want).max() <= 2e-3 * max(1.0, np.abs(y).max())


def test_mlp_block_rejects_bad_arguments(lib):
    import ctypes

    one = ctypes.c_void_p(0x1000)
    f = lib.launch_nvfp4_mlp_tc
    assert f(one, one, one, one, one, one, one, 1e-6, 512, 200, None) == -2      # hidden % 256
    assert f(one, one, one, one, one, one, one, 1e-6, 500, 256, None) == -2      # inter % 256
    assert f(one, one, one, one, one, one, None, 1e-6, 512, 256, None) == -2     # norm weights missing
    assert f(one, one, one, one, one, one, one, 1e-6, 512, 12288, None) == -2    # hidden > 11520

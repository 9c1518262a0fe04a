"""GEMV parity on the GPU, through the C ABI, against the CPU oracle.

Tolerance (fp32 accumulation of exact products): max over outputs of
|y - ref| / max(|ref|, 1e-3 * max|ref|) <= 1e-3, ref = float64 product of the exactly decoded
matrix; fp16 rounding of the result alone accounts for up to 4.9e-4.  The reference's own GEMM
acceptance rule (mean_rel < 0.01, max_abs < max(0.1, 1% max|ref|)) is checked as a floor.
"""
import numpy as np
import pytest

from oracle import nvfp4_codec_oracle as oc
from tests.gpu_util import gemv, gemv2, gemv2i

pytestmark = pytest.mark.gpu

TOL = 1e-3


def check(y, packed, scales, act):
    ref = oc.gemv_f64(packed, scales, act)
    rel = oc.rel_error_floored(y, ref)
    assert np.isfinite(y.astype(np.float64)).all()
    assert rel.max() <= TOL, f"max rel {rel.max():.3e}"
    # the correctly rounded result is reachable: most outputs are the nearest fp16
    exact = (y == ref.astype(np.float16)).mean()
    assert exact > 0.95, exact
    ok, mean_rel, max_abs = oc.reference_gemm_check(y, ref)
    assert ok, (mean_rel, max_abs)


def test_golden_fixture(lib, golden):
    rc, y = gemv(lib, golden["gemv_packed"], golden["gemv_scales"], golden["gemv_act"])
    assert rc == 0
    check(y, golden["gemv_packed"], golden["gemv_scales"], golden["gemv_act"])
    assert oc.rel_error_floored(y, golden["gemv_y_f32"]).max() <= TOL


@pytest.mark.parametrize("M,K", [
    (1, 128), (7, 128), (16, 256), (48, 5120), (100, 768), (17, 384), (1024, 5120),
    (33, 17408), (5120, 5120), (257, 6144),
])
def test_shapes_tensor_core_path(lib, M, K):
    w = oc.synthetic_weight(M, K, seed=M * 31 + K)
    p, s = oc.encode(w)
    a = oc.synthetic_act(K, seed=K)
    rc, y = gemv(lib, p, s, a)
    assert rc == 0
    check(y, p, s, a)


@pytest.mark.parametrize("M,K", [(1, 32), (7, 96), (48, 160), (100, 5152), (9, 32 * 7)])
def test_shapes_generic_path(lib, M, K):
    # K % 32 == 0 but K % 128 != 0: served by the non-tensor-core kernel
    w = oc.synthetic_weight(M, K, seed=M + K)
    p, s = oc.encode(w)
    a = oc.synthetic_act(K, seed=K + 5)
    rc, y = gemv(lib, p, s, a)
    assert rc == 0
    check(y, p, s, a)


def test_every_entry_point_agrees(lib):
    w = oc.synthetic_weight(64, 640, seed=11)
    p, s = oc.encode(w)
    a = oc.synthetic_act(640, seed=12)
    base = None
    for entry in ("launch_nvfp4_gemv", "launch_nvfp4_gemv_v8", "launch_nvfp4_gemv_v4",
                  "launch_nvfp4_gemv_v5", "launch_nvfp4_gemv_v6", "launch_nvfp4_gemv_v7",
                  "launch_nvfp4_gemvnl"):
        rc, y = gemv(lib, p, s, a, entry=entry)
        assert rc == 0, entry
        if base is None:
            base = y
        assert np.array_equal(base.view(np.uint16), y.view(np.uint16)), entry


def test_both_kernels_agree_and_config_hook(lib):
    w = oc.synthetic_weight(200, 1024, seed=21)
    p, s = oc.encode(w)
    a = oc.synthetic_act(1024, seed=22)
    outs = []
    try:
        for cfg in ((0, 0, 0), (2, 0, 0), (4, 1, 0), (8, 0, 0), (0, 0, 1), (0, 0, 2),
                    (4, 0, 0x200), (8, 0, 0x400), (4, 2, 0x200), (8, 1, 0x402), (4, 0, 0x100), (0, 0, 0x10)):
            assert lib.nvfp4_b200_gemv_config(*cfg) == 0
            rc, y = gemv(lib, p, s, a)
            assert rc == 0
            check(y, p, s, a)
            outs.append(y)
    finally:
        lib.nvfp4_b200_gemv_config(0, 0, 0)
    for y in outs[1:]:
        # different summation orders: equal to within one fp16 step
        assert oc.rel_error_floored(y, outs[0].astype(np.float64)).max() <= 1e-3


@pytest.mark.parametrize("flags", [0x200, 0x400])
@pytest.mark.parametrize("M,K", [(1, 128), (100, 768), (257, 6144), (33, 17408), (1024, 5120)])
def test_cluster_split_k(lib, M, K, flags):
    # row tiles shared by a cluster of 2 or 4 CTAs (partial sums combined through distributed
    # shared memory), incl. ragged rows, K % 256 != 0 and more CTAs than K steps
    w = oc.synthetic_weight(M, K, seed=M * 7 + K)
    p, s = oc.encode(w)
    a = oc.synthetic_act(K, seed=K + 1)
    try:
        for warps in (4, 8):
            assert lib.nvfp4_b200_gemv_config(warps, 0, flags) == 0
            rc, y = gemv(lib, p, s, a)
            assert rc == 0
            check(y, p, s, a)
            a2 = oc.synthetic_act(K, seed=K + 2)
            rc, y2 = gemv2(lib, p, s, a, a2)
            assert rc == 0
            check(y2[0], p, s, a)
            check(y2[1], p, s, a2)
    finally:
        lib.nvfp4_b200_gemv_config(0, 0, 0)


def test_mixed_magnitude_scales(lib):
    # blocks whose scale bytes span a wide range, including all-zero blocks (byte 127)
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((64, 512)) * rng.choice([1e-4, 0.02, 1.0, 300.0], (64, 512 // 16)).repeat(16, axis=1)).astype(np.float16)
    w[3, 32:48] = 0
    w[5] = 0
    p, s = oc.encode(w)
    assert s.min() < 116 and s.max() > 130
    a = oc.synthetic_act(512, seed=9)
    rc, y = gemv(lib, p, s, a)
    assert rc == 0
    check(y, p, s, a)
    assert y[5] == 0


def test_scale_byte_extremes(lib):
    # byte 0 decodes to +0 scale (as in the reference kernels, which build the fp32 exponent
    # directly) and large bytes overflow fp16 to inf without faulting
    p = np.full((16, 64), 0x22, dtype=np.uint8)        # every weight = +1.0
    s = np.full((16, 8), 127, dtype=np.uint8)
    s[1, :] = 0
    s[2, :] = 254
    a = np.ones(128, dtype=np.float16)
    rc, y = gemv(lib, p, s, a)
    assert rc == 0
    assert y[0] == 128 and y[1] == 0 and np.isinf(y[2]) and y[3] == 128


def test_linearity_full_size(lib):
    # size-independent property at a full 27B layer shape: W(a+b) = Wa + Wb when a, b and a+b
    # are exactly representable (small integers), so all three GEMVs are exact in fp32
    M, K = 17408, 5120
    rng = np.random.default_rng(1)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = np.full((M, K // 16), 127 - 4, dtype=np.uint8)
    a = rng.integers(-2, 3, size=K).astype(np.float16)
    b = rng.integers(-2, 3, size=K).astype(np.float16)
    _, ya = gemv(lib, p, s, a)
    _, yb = gemv(lib, p, s, b)
    _, yab = gemv(lib, p, s, a + b)
    ref = oc.gemv_f64(p, s, a + b)
    assert np.array_equal(yab.astype(np.float64), ref.astype(np.float16).astype(np.float64))
    ra, rb = oc.gemv_f64(p, s, a), oc.gemv_f64(p, s, b)
    assert np.array_equal(ya.astype(np.float64), ra.astype(np.float16).astype(np.float64))
    assert np.array_equal(yb.astype(np.float64), rb.astype(np.float16).astype(np.float64))


def test_gemv2_two_activations(lib):
    for M, K in ((48, 256), (100, 5120), (31, 96)):
        w = oc.synthetic_weight(M, K, seed=M)
        p, s = oc.encode(w)
        a0, a1 = oc.synthetic_act(K, seed=1), oc.synthetic_act(K, seed=2)
        rc, y = gemv2(lib, p, s, a0, a1)
        assert rc == 0
        check(y[0], p, s, a0)
        check(y[1], p, s, a1)


def test_gemv2i_interleaved_activations(lib):
    # reference: kernels/nvfp4_gemv.cu:997-1011; shapes cover the tensor-core kernel with 4 and 8
    # warps, the generic kernel (K % 128 != 0) and a ragged last row tile
    for M, K in ((48, 256), (100, 5120), (31, 96), (5120, 6144), (1030, 17408)):
        w = oc.synthetic_weight(M, K, seed=M + 3)
        p, s = oc.encode(w)
        a0, a1 = oc.synthetic_act(K, seed=5), oc.synthetic_act(K, seed=6)
        rc, y = gemv2i(lib, p, s, a0, a1)
        assert rc == 0
        check(y[0], p, s, a0)
        check(y[1], p, s, a1)
        rc2, y2 = gemv2(lib, p, s, a0, a1)
        assert rc2 == 0 and np.array_equal(y.view(np.uint16), y2.view(np.uint16))
    assert lib.launch_nvfp4_gemv2i(None, None, None, None, 16, 48, None) == -2


def test_config1_full_size(lib):
    # the single-GEMV workload: W [5120, 5120] ~ N(0, 0.02^2), x ~ N(0, 1)
    w = oc.synthetic_weight(5120, 5120, seed=0)
    p, s = oc.encode(w)
    a = oc.synthetic_act(5120, seed=0)
    rc, y = gemv(lib, p, s, a)
    assert rc == 0
    check(y, p, s, a)

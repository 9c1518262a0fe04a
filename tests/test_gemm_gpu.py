"""Dense NVFP4 GEMM (launch_nvfp4_gemmtc_v5) on the GPU against the CPU oracle.

Oracle: the reference's truth recipe — decode the weights to fp16 with the codec, multiply with
the fp16 activations (simulation/nvfp4_cuda_v5_test.py:90-91), here in float64.  Tolerances: the
reference's own acceptance rule (mean_rel < 0.01 and max_abs < max(0.1, 1 % of max|ref|),
simulation/nvfp4_cuda_v5_test.py:92-95,186) and, tighter, max |y - ref| / max(|ref|, 1e-3 max|ref|)
<= 2e-3 * max(1, sqrt(K / 4096)) (fp32 accumulation in tensor memory; fp16 output rounding alone
is 4.9e-4)."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_codec_oracle as oc
from tests.gpu_util import dev, ptr, stream

pytestmark = pytest.mark.gpu


def run_gemm(lib, packed, scales, act_kn):
    M, K = packed.shape[0], packed.shape[1] * 2
    N = act_kn.shape[1]
    d_p, d_s, d_a = dev(packed), dev(scales), dev(act_kn.astype(np.float16))
    out = torch.full((M * N + 16,), float("nan"), dtype=torch.float16, device="cuda")
    rc = lib.launch_nvfp4_gemmtc_v5(ptr(d_p), ptr(d_s), ptr(d_a), ptr(out), M, N, K, stream())
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.isnan(o[M * N:]).all(), "wrote past the output"
    return rc, o[:M * N].reshape(M, N)


def check(y, packed, scales, act_kn):
    w = oc.decode(packed, scales).astype(np.float64)
    ref = w @ act_kn.astype(np.float16).astype(np.float64)
    assert np.isfinite(y.astype(np.float64)).all()
    ok, mean_rel, max_abs = oc.reference_gemm_check(y, ref)
    assert ok, (mean_rel, max_abs)
    rel = oc.rel_error_floored(y, ref)
    K = act_kn.shape[0]
    # the tensor core's fp32 accumulation error grows with the number of terms
    assert rel.max() <= 2e-3 * max(1.0, (K / 4096) ** 0.5), rel.max()


@pytest.mark.parametrize("M,N,K", [
    (128, 64, 64), (128, 128, 256), (256, 8, 128), (300, 200, 512), (100, 24, 320),
    (1024, 512, 5120), (512, 256, 16384), (17408, 32, 5120), (5120, 136, 6144),
])
def test_tensor_core_path(lib, M, N, K):
    lib.nvfp4_gemm_status(1)
    w = oc.synthetic_weight(M, K, seed=M + N + K)
    p, s = oc.encode(w)
    a = np.random.default_rng(N).standard_normal((K, N)).astype(np.float16)
    rc, y = run_gemm(lib, p, s, a)
    assert rc == 0
    assert lib.nvfp4_gemm_status(0) == 0, "a bounded wait inside the kernel ran out"
    check(y, p, s, a)


@pytest.mark.parametrize("M,N,K", [(100, 100, 112), (7, 3, 16), (64, 33, 64), (33, 8, 48)])
def test_fallback_path(lib, M, N, K):
    # the reference's boundary shape 100 x 100 x 112 and other shapes the tensor-core kernel
    # does not take (K % 64 != 0 or N % 8 != 0)
    w = oc.synthetic_weight(M, K, seed=M * K)
    p, s = oc.encode(w)
    a = np.random.default_rng(K).standard_normal((K, N)).astype(np.float16)
    rc, y = run_gemm(lib, p, s, a)
    assert rc == 0
    check(y, p, s, a)


def test_matches_gemv_column_by_column(lib):
    # a GEMM over N tokens equals N GEMVs up to the fp16-scaled-weight rounding of the W4A16 path
    from tests.gpu_util import gemv

    M, N, K = 256, 16, 1024
    w = oc.synthetic_weight(M, K, seed=5)
    p, s = oc.encode(w)
    a = np.random.default_rng(6).standard_normal((K, N)).astype(np.float16)
    rc, y = run_gemm(lib, p, s, a)
    assert rc == 0
    for n in (0, 7, 15):
        rc, yv = gemv(lib, p, s, np.ascontiguousarray(a[:, n]))
        assert rc == 0
        assert oc.rel_error_floored(y[:, n], yv.astype(np.float64)).max() <= 2e-3


def test_argument_validation(lib):
    import ctypes

    one = ctypes.c_void_p(0x1000)
    assert lib.launch_nvfp4_gemmtc_v5(one, one, one, one, 16, 8, 24, None) == -2   # K % 16
    assert lib.launch_nvfp4_gemmtc_v5(one, one, one, one, 0, 8, 64, None) == -2
    assert lib.launch_nvfp4_gemmtc_v5(None, one, one, one, 16, 8, 64, None) == -2
    assert lib.get_kernel_shared_mem_bytes() > 64 * 1024


def test_w4a4_activation_quantisation_and_product(lib):
    # W4A4 semantics (both operands in the block-16 E8M0 format): activations quantised per 16-element block along K with
    # the codec, both operands dequantised, fp32-accumulated product.  Oracle: the codec on the
    # CPU for both operands, float64 matmul.
    import ctypes

    rng = np.random.default_rng(5)
    for M, n, K in ((256, 32, 512), (384, 13, 1024), (128, 70, 5120)):
        w = oc.synthetic_weight(M, K, seed=M + n)
        p, s = oc.encode(w)
        act = rng.standard_normal((n, K)).astype(np.float16)
        act[0, :16] = 0
        act[1 % n, 16:32] *= 100
        ap, asc = oc.encode(act)
        aq = oc.decode_f64(ap, asc)                                  # [n, K]
        N = (n + 7) // 8 * 8
        d_act = torch.from_numpy(act).cuda()
        work = torch.full((K * N + 8,), 9.0, dtype=torch.float16, device="cuda")
        rc = lib.launch_nvfp4_quant_dequant_T(ptr(d_act), K, ptr(work), N, n, K, stream())
        torch.cuda.synchronize()
        assert rc == 0
        got = work.cpu().numpy()
        assert (got[K * N:] == 9.0).all()
        got = got[:K * N].reshape(K, N)
        assert np.array_equal(got[:, :n].astype(np.float64), aq.T) and (got[:, n:] == 0).all()

        d_p, d_s = torch.from_numpy(p).cuda(), torch.from_numpy(s).cuda()
        out = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        rc = lib.launch_nvfp4_gemm_w4a4(ptr(d_p), ptr(d_s), ptr(d_act), ptr(out), ptr(work), M, n, K,
                                        stream())
        torch.cuda.synchronize()
        assert rc == 0 and lib.nvfp4_gemm_status(0) == 0
        ref = oc.decode_f64(p, s) @ aq.T                              # [M, n]
        y = out.cpu().numpy()[:, :n]
        assert oc.rel_error_floored(y, ref).max() <= 2e-3 * max(1.0, (K / 4096) ** 0.5), (M, n, K)
    assert lib.launch_nvfp4_gemm_w4a4(ptr(d_p), ptr(d_s), ptr(d_act), ptr(out), None, M, n, K,
                                      stream()) == -2


def assert_doubled(y2, y):
    # y2 == 2 y exactly wherever y was rounded to 11 significant bits; below 2^-13 (subnormals, and
    # the lowest binade, which a subnormal-range value can round up into) y sits on the fixed
    # 2^-24 grid, coarser relative to it than to its double: there they may differ by one step
    y, y2 = y.float(), y2.float()
    normal = y.abs() >= 2.0 ** -13
    assert bool(torch.where(normal, y2 == 2 * y, (y2 - 2 * y).abs() <= 2.0 ** -23).all())


@pytest.mark.parametrize("M,n,K", [
    (128, 32, 256), (256, 32, 512), (384, 13, 1024), (128, 70, 5120), (300, 200, 512),
    (1024, 512, 5120), (200, 136, 6144), (640, 1000, 1024),
])
def test_fp4_block_scaled_tensor_core_path(lib, M, n, K):
    # both operands as NVFP4 bytes straight into tcgen05.mma kind::mxf4nvf4 (block-16 E8M0 scales).
    # Oracle: the codec's decode of both byte sets on the CPU, float64 product.  Every nibble
    # product and scale product is exact, so only the fp32 accumulation and the fp16 output round.
    rng = np.random.default_rng(M + n + K)
    w = oc.synthetic_weight(M, K, seed=M + K)
    p, s = oc.encode(w)
    act = rng.standard_normal((n, K)).astype(np.float16)
    act[0, :16] = 0                                     # an all-zero block
    act[n // 2, 16:32] *= 50                            # a block with a large scale
    ap, asc = oc.encode(act)
    d_p, d_s, d_ap, d_as = dev(p), dev(s), dev(ap), dev(asc)
    ld = (n + 7) // 8 * 8
    out = torch.full((M * ld + 16,), float("nan"), dtype=torch.float16, device="cuda")
    lib.nvfp4_gemm_fp4_status(1)
    rc = lib.launch_nvfp4_gemm_fp4(ptr(d_p), ptr(d_s), ptr(d_ap), ptr(d_as), ptr(out), M, n, K, ld,
                                   stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert lib.nvfp4_gemm_fp4_status(0) == 0, "a bounded wait inside the kernel ran out"
    o = out.cpu().numpy()
    assert np.isnan(o[M * ld:]).all(), "wrote past the output"
    y = o[:M * ld].reshape(M, ld)[:, :n]
    ref = oc.decode_f64(p, s) @ oc.decode_f64(ap, asc).T
    assert np.isfinite(y.astype(np.float64)).all()
    assert oc.rel_error_floored(y, ref).max() <= 2e-3 * max(1.0, (K / 4096) ** 0.5)
    # device-side quantiser + FP4 product through the one-call entry equals the same oracle
    N = ld
    d_act = torch.from_numpy(act).cuda()
    work = torch.zeros(K * N, dtype=torch.float16, device="cuda")
    out2 = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    rc = lib.launch_nvfp4_gemm_w4a4(ptr(d_p), ptr(d_s), ptr(d_act), ptr(out2), ptr(work), M, n, K,
                                    stream())
    torch.cuda.synchronize()
    assert rc == 0 and lib.nvfp4_gemm_status(0) == 0
    assert np.array_equal(out2.cpu().numpy()[:, :n], y)


def test_fp4_prefill_size_8192_tokens(lib):
    # 17408 x 5120 weights, 8192 tokens; oracle on a sample of rows and tokens (see the W4A16
    # test below), plus exact linearity in the scale bytes over the WHOLE output: raising every
    # activation scale byte by one doubles every output exactly
    M, K, tokens = 17408, 5120, 8192
    rng = np.random.default_rng(7)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
    ap = rng.integers(0, 256, size=(tokens, K // 2), dtype=np.uint8)
    asc = rng.integers(122, 127, size=(tokens, K // 16), dtype=np.uint8)
    d_p, d_s, d_ap, d_as = dev(p), dev(s), dev(ap), dev(asc)
    out = torch.full((M * tokens + 16,), float("nan"), dtype=torch.float16, device="cuda")
    lib.nvfp4_gemm_fp4_status(1)
    rc = lib.launch_nvfp4_gemm_fp4(ptr(d_p), ptr(d_s), ptr(d_ap), ptr(d_as), ptr(out), M, tokens, K,
                                   tokens, stream())
    torch.cuda.synchronize()
    assert rc == 0 and lib.nvfp4_gemm_fp4_status(0) == 0
    assert bool(torch.isnan(out[M * tokens:]).all()), "wrote past the output"
    y = out[:M * tokens].view(M, tokens)
    assert bool(torch.isfinite(y).all())
    rows = np.unique(np.concatenate([[0, M - 1], rng.integers(0, M, 62)]))
    cols = np.unique(np.concatenate([[0, tokens - 1], rng.integers(0, tokens, 94)]))
    ref = oc.decode_f64(p[rows], s[rows]) @ oc.decode_f64(ap[cols], asc[cols]).T
    got = y[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy()
    assert oc.rel_error_floored(got, ref).max() <= 2e-3 * max(1.0, (K / 4096) ** 0.5)
    d_as2 = d_as + 1
    out2 = torch.empty(M * tokens, dtype=torch.float16, device="cuda")
    assert lib.launch_nvfp4_gemm_fp4(ptr(d_p), ptr(d_s), ptr(d_ap), ptr(d_as2), ptr(out2), M, tokens,
                                     K, tokens, stream()) == 0
    torch.cuda.synchronize()
    assert_doubled(out2.view(M, tokens), y)


@pytest.mark.parametrize("M,n,K", [(5120, 32, 17408), (640, 64, 10240), (300, 100, 10240), (1000, 7, 12288),
                                   (200, 136, 16384)])
def test_fp4_batched_decode_splits_k(lib, M, n, K):
    # batched decode (32 tokens) of a down projection: 40 output tiles of 68 K stages would leave
    # two thirds of the SMs idle, so K (>= 40 stages of 256) is split over several CTAs per tile
    # and the last to arrive adds the fp32 partial tiles in split order.  Oracle as above over the whole output; the split result is reproducible bit
    # for bit (the order of the sum does not depend on which CTA comes last), and differs from
    # the unsplit kernel's only by the fp32 association of the K sum.
    rng = np.random.default_rng(M + n)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
    ap = rng.integers(0, 256, size=(n, K // 2), dtype=np.uint8)
    asc = rng.integers(122, 127, size=(n, K // 16), dtype=np.uint8)
    d_p, d_s, d_ap, d_as = dev(p), dev(s), dev(ap), dev(asc)
    ld = (n + 7) // 8 * 8
    ref = oc.decode_f64(p, s) @ oc.decode_f64(ap, asc).T
    tol = 2e-3 * max(1.0, (K / 4096) ** 0.5)

    def run():
        out = torch.full((M * ld + 16,), float("nan"), dtype=torch.float16, device="cuda")
        rc = lib.launch_nvfp4_gemm_fp4(ptr(d_p), ptr(d_s), ptr(d_ap), ptr(d_as), ptr(out), M, n, K,
                                       ld, stream())
        torch.cuda.synchronize()
        assert rc == 0 and lib.nvfp4_gemm_fp4_status(0) == 0
        o = out.cpu().numpy()
        assert np.isnan(o[M * ld:]).all(), "wrote past the output"
        return o[:M * ld].reshape(M, ld)[:, :n]

    lib.nvfp4_gemm_fp4_status(1)
    try:
        ys = [run() for _ in range(3)]
        lib.nvfp4_b200_gemm_fp4_config(0)
        y1 = run()
    finally:
        lib.nvfp4_b200_gemm_fp4_config(3)
    for y in ys + [y1]:
        assert np.isfinite(y.astype(np.float64)).all()
        assert oc.rel_error_floored(y, ref).max() <= tol
    assert np.array_equal(ys[0], ys[1]) and np.array_equal(ys[0], ys[2])
    assert oc.rel_error_floored(ys[0], y1.astype(np.float64)).max() <= tol


@pytest.mark.parametrize("M,K", [(17408, 5120), (5120, 17408)])
def test_prefill_size_8192_tokens(lib, M, K):
    # the prefill workload (4 sequences x 2048 tokens): 32 token tiles of 256 per row tile.  The
    # float64 oracle of the whole product would take minutes, so it is evaluated on a sample:
    # 64 weight rows spread over the matrix (every row tile position) x 96 tokens spread over the
    # token range (every token tile), plus the first and last row and token.
    tokens = 8192
    rng = np.random.default_rng(M)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
    d_a = (torch.randn(K, tokens, device="cuda", generator=torch.Generator("cuda").manual_seed(K))
           ).to(torch.float16)
    d_p, d_s = dev(p), dev(s)
    out = torch.full((M * tokens + 16,), float("nan"), dtype=torch.float16, device="cuda")
    lib.nvfp4_gemm_status(1)
    rc = lib.launch_nvfp4_gemmtc_v5(ptr(d_p), ptr(d_s), ptr(d_a), ptr(out), M, tokens, K, stream())
    torch.cuda.synchronize()
    assert rc == 0 and lib.nvfp4_gemm_status(0) == 0
    assert bool(torch.isnan(out[M * tokens:]).all()), "wrote past the output"
    y = out[:M * tokens].view(M, tokens)
    assert bool(torch.isfinite(y).all())
    rows = np.unique(np.concatenate([[0, M - 1], rng.integers(0, M, 62)]))
    cols = np.unique(np.concatenate([[0, tokens - 1], rng.integers(0, tokens, 94)]))
    w = oc.decode(p[rows], s[rows]).astype(np.float64)
    a = d_a[:, torch.from_numpy(cols).cuda()].cpu().numpy().astype(np.float64)
    ref = w @ a
    got = y[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy()
    ok, mean_rel, max_abs = oc.reference_gemm_check(got, ref)
    assert ok, (mean_rel, max_abs)
    assert oc.rel_error_floored(got, ref).max() <= 2e-3 * max(1.0, (K / 4096) ** 0.5)
    # linearity as a size-independent property over the WHOLE output: doubling the activations
    # doubles every output exactly (powers of two commute with every rounding)
    d_a2 = d_a * 2
    out2 = torch.empty(M * tokens, dtype=torch.float16, device="cuda")
    assert lib.launch_nvfp4_gemmtc_v5(ptr(d_p), ptr(d_s), ptr(d_a2), ptr(out2), M, tokens, K,
                                      stream()) == 0
    torch.cuda.synchronize()
    assert_doubled(out2.view(M, tokens), y)


def test_against_the_reference_gemm_kernel(lib):
    # the reference's own wmma kernel, recompiled unchanged (oracle/_ref), beside ours on the same
    # bytes: both implement W4A16 (weight x scale in fp16, fp16 products, fp32 accumulation), so
    # they agree to accumulation-order noise, and both meet the reference's acceptance rule
    import ctypes
    import os

    from conftest import ROOT

    path = os.path.join(ROOT, "oracle", "_ref", "ref_nvfp4_cuda_v5.so")
    if not os.path.exists(path):
        pytest.skip(f"{path} not built (needs the reference tree: make -C oracle REF=...)")
    ref = ctypes.CDLL(path)
    for M, N, K in ((256, 64, 512), (1024, 512, 5120), (100, 100, 112)):
        w = oc.synthetic_weight(M, K, seed=M + K)
        p, s = oc.encode(w)
        a = np.random.default_rng(N).standard_normal((K, N)).astype(np.float16)
        d_p, d_s, d_a = dev(p), dev(s), dev(a)
        outs = []
        for L in (lib, ref):
            o = torch.zeros((M, N), dtype=torch.float16, device="cuda")
            rc = L.launch_nvfp4_gemmtc_v5(ptr(d_p), ptr(d_s), ptr(d_a), ptr(o), M, N, K, stream())
            torch.cuda.synchronize()
            assert rc == 0
            outs.append(o.cpu().numpy())
        truth = oc.decode(p, s).astype(np.float64) @ a.astype(np.float64)
        for y in outs:
            assert oc.reference_gemm_check(y, truth)[0]
        assert oc.rel_error_floored(outs[0], outs[1].astype(np.float64)).max() <= 4e-3


@pytest.mark.parametrize("M,n,K", [
    (256, 64, 512), (1000, 13, 1024), (640, 100, 2048), (640, 200, 6144), (5120, 512, 5120),
    (17408, 512, 5120), (5120, 509, 8704),
])
def test_token_major_entry_equals_transposing_around_the_gemm(lib, M, n, K):
    # launch_nvfp4_gemm_w4a16_ex reads token-major activations as a K-major B operand and / or
    # writes token-major (optionally adding into the output, the decoder's residual add): the same
    # MMAs in the same order as launch_nvfp4_gemmtc_v5, so every combination is bit-identical to
    # transposing around that call.  The plain call itself is checked against the oracle above;
    # here also directly for the all-token-major combination.
    rng = np.random.default_rng(M + n + K)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
    act = rng.standard_normal((n, K)).astype(np.float16)          # token-major
    N8 = (n + 7) // 8 * 8
    d_p, d_s = dev(p), dev(s)
    a_tm = torch.from_numpy(act).cuda()
    a_fm = torch.zeros((K, N8), dtype=torch.float16, device="cuda")
    a_fm[:, :n] = a_tm.t()
    base = torch.zeros((M, N8), dtype=torch.float16, device="cuda")
    lib.nvfp4_gemm_status(1)
    assert lib.launch_nvfp4_gemmtc_v5(ptr(d_p), ptr(d_s), ptr(a_fm), ptr(base), M, N8, K, stream()) == 0
    torch.cuda.synchronize()
    want_fm = base[:, :n].clone()
    want_tm = want_fm.t().contiguous()
    resid = torch.from_numpy(rng.standard_normal((n, M)).astype(np.float16)).cuda()
    want_add = (resid.float() + want_tm.float()).half()
    pitch = M + 24                                               # an output pitch wider than M
    for in_tm in (0, 1):
        a, ld_a = (a_tm, K) if in_tm else (a_fm, N8)
        out = torch.full((M * N8 + 16,), float("nan"), dtype=torch.float16, device="cuda")
        assert lib.launch_nvfp4_gemm_w4a16_ex(ptr(d_p), ptr(d_s), ptr(a), ld_a, ptr(out), N8, M, n, K,
                                              in_tm, stream()) == 0
        torch.cuda.synchronize()
        assert bool(torch.isnan(out[M * N8:]).all()), "wrote past the output"
        got = out[:M * N8].view(M, N8)
        assert torch.equal(got[:, :n], want_fm)
        assert bool((got[:, n:] == 0).all())
        out = torch.full((n * pitch + 16,), float("nan"), dtype=torch.float16, device="cuda")
        assert lib.launch_nvfp4_gemm_w4a16_ex(ptr(d_p), ptr(d_s), ptr(a), ld_a, ptr(out), pitch, M, n,
                                              K, in_tm | 2, stream()) == 0
        torch.cuda.synchronize()
        got = out[:n * pitch].view(n, pitch)
        assert torch.equal(got[:, :M], want_tm)
        assert bool(torch.isnan(got[:, M:]).all()) and bool(torch.isnan(out[n * pitch:]).all())
        acc = resid.clone()
        assert lib.launch_nvfp4_gemm_w4a16_ex(ptr(d_p), ptr(d_s), ptr(a), ld_a, ptr(acc), M, M, n, K,
                                              in_tm | 2 | 4, stream()) == 0
        torch.cuda.synchronize()
        assert torch.equal(acc, want_add)
    assert lib.nvfp4_gemm_status(0) == 0
    if M * n <= 1 << 20:
        check(want_tm.t().cpu().numpy(), p, s, act.T)


def test_token_major_entry_argument_validation(lib):
    z = torch.zeros(1 << 16, dtype=torch.float16, device="cuda")
    b = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    st = stream()
    ok = lambda *a: lib.launch_nvfp4_gemm_w4a16_ex(*a, st)
    assert ok(ptr(b), ptr(b), ptr(z), 64, ptr(z), 128, 128, 16, 64, 3) == 0
    assert ok(ptr(b), ptr(b), ptr(z), 64, ptr(z), 128, 128, 16, 48, 3) == -2      # K % 64
    assert ok(ptr(b), ptr(b), ptr(z), 60, ptr(z), 128, 128, 16, 64, 3) == -2      # ld_act % 8 / < K
    assert ok(ptr(b), ptr(b), ptr(z), 64, ptr(z), 100, 128, 16, 64, 3) == -2      # ld_out < M
    assert ok(ptr(b), ptr(b), ptr(z), 64, ptr(z), 128, 128, 16, 64, 4) == -2      # add without token-major out
    assert ok(ptr(b), ptr(b), ptr(z), 24, ptr(z), 16, 128, 13, 64, 0) == -2       # feature-major pitch != 16
    assert ok(ptr(b), ptr(b), ptr(z), 16, ptr(z), 16, 128, 13, 64, 0) == 0
    assert ok(ptr(b), ptr(b), None, 64, ptr(z), 128, 128, 16, 64, 3) == -2
    assert ok(ptr(b), ptr(b), ptr(z), 64, ptr(z), 128, 128, 16, 64, 8) == -2
    torch.cuda.synchronize()


@pytest.mark.parametrize("M,n,K", [
    (300, 136, 512), (640, 200, 2048), (5120, 512, 5120), (17408, 512, 5120), (5120, 509, 8704),
    (1000, 1000, 1024),
])
def test_cta_pair_kernel_equals_the_single_cta_kernel(lib, M, n, K):
    # the CTA-pair kernel (clusters of two, one M = 256 MMA on both SMs' tensor cores, each CTA
    # holding half of the token tile) adds the same products in the same K order: every layout
    # combination is bit-identical to the single-CTA kernel, which the tests above pin to the oracle
    rng = np.random.default_rng(M * 3 + n + K)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
    act = rng.standard_normal((n, K)).astype(np.float16)
    N8 = (n + 7) // 8 * 8
    d_p, d_s = dev(p), dev(s)
    a_tm = torch.from_numpy(act).cuda()
    a_fm = torch.zeros((K, N8), dtype=torch.float16, device="cuda")
    a_fm[:, :n] = a_tm.t()
    resid = torch.from_numpy(rng.standard_normal((n, M)).astype(np.float16)).cuda()

    def run_all():
        outs = []
        o = torch.full((M * N8 + 16,), float("nan"), dtype=torch.float16, device="cuda")
        assert lib.launch_nvfp4_gemmtc_v5(ptr(d_p), ptr(d_s), ptr(a_fm), ptr(o), M, N8, K, stream()) == 0
        outs.append(o)
        for flags in (1, 2, 3, 6, 7):
            a, ld_a = (a_tm, K) if flags & 1 else (a_fm, N8)
            if flags & 2:
                o = resid.clone() if flags & 4 else torch.full((n * M + 16,), float("nan"),
                                                               dtype=torch.float16, device="cuda")
                ld_o = M
            else:
                o = torch.full((M * N8 + 16,), float("nan"), dtype=torch.float16, device="cuda")
                ld_o = N8
            assert lib.launch_nvfp4_gemm_w4a16_ex(ptr(d_p), ptr(d_s), ptr(a), ld_a, ptr(o), ld_o, M, n, K,
                                                  flags, stream()) == 0
            outs.append(o)
        torch.cuda.synchronize()
        assert lib.nvfp4_gemm_status(0) == 0, "a bounded wait inside the kernel ran out"
        return outs

    lib.nvfp4_gemm_status(1)
    try:
        lib.nvfp4_b200_gemm_config(1)          # single-CTA kernels only
        want = run_all()
        lib.nvfp4_b200_gemm_config(7)          # the pair kernel for every shape
        got = run_all()
    finally:
        lib.nvfp4_b200_gemm_config(3)
    for w, g in zip(want, got):
        assert torch.equal(torch.nan_to_num(w, nan=12345.0), torch.nan_to_num(g, nan=12345.0))


@pytest.mark.parametrize("M,n,K", [(300, 136, 512), (1024, 512, 5120), (640, 1000, 1024), (5120, 509, 8704),
                                   (384, 200, 12288)])
def test_fp4_cta_pair_kernel_equals_the_single_cta_kernel(lib, M, n, K):
    # more than 128 tokens run on clusters of two CTAs (one M = 256 block-scaled MMA on both SMs'
    # tensor cores, each CTA holding half of the token tile): same products, same K order, so the
    # output is bit-identical to the single-CTA kernel's, which the tests above pin to the oracle
    rng = np.random.default_rng(M + 7 * n + K)
    p = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    s = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
    ap = rng.integers(0, 256, size=(n, K // 2), dtype=np.uint8)
    asc = rng.integers(122, 127, size=(n, K // 16), dtype=np.uint8)
    d_p, d_s, d_ap, d_as = dev(p), dev(s), dev(ap), dev(asc)
    ld = (n + 7) // 8 * 8
    outs = []
    lib.nvfp4_gemm_fp4_status(1)
    try:
        for cfg in (1, 7):                       # single-CTA kernel, then the pair kernel for every K
            lib.nvfp4_b200_gemm_fp4_config(cfg)
            out = torch.full((M * ld + 16,), float("nan"), dtype=torch.float16, device="cuda")
            assert lib.launch_nvfp4_gemm_fp4(ptr(d_p), ptr(d_s), ptr(d_ap), ptr(d_as), ptr(out), M, n, K,
                                             ld, stream()) == 0
            torch.cuda.synchronize()
            assert lib.nvfp4_gemm_fp4_status(0) == 0, "a bounded wait inside the kernel ran out"
            assert bool(torch.isnan(out[M * ld:]).all()), "wrote past the output"
            outs.append(out[:M * ld].view(M, ld)[:, :n].clone())
    finally:
        lib.nvfp4_b200_gemm_fp4_config(3)
    assert bool(torch.isfinite(outs[0]).all())
    assert torch.equal(outs[0], outs[1])
    if M * n <= 1 << 19:
        ref = oc.decode_f64(p, s) @ oc.decode_f64(ap, asc).T
        assert oc.rel_error_floored(outs[1].cpu().numpy(), ref).max() <= 2e-3 * max(1.0, (K / 4096) ** 0.5)

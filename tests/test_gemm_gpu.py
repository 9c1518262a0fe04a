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

"""The allocation-free DeltaNet entry point against the regular one, through the C ABI.

`launch_dn_fused_noalloc` is for callers that cannot call cudaMalloc where they launch the step
(all device memory already belongs to another allocator, or the stream is being captured): the
workspace between the step's two kernels is a 40 KB array inside the library instead of a buffer
the caller passes.  Both entry points run the same kernels, so from identical inputs they must
produce identical bytes; the check is repeated for two consecutive calls because the second call
reuses a workspace that still holds the first call's values.

This file sorts last on purpose: a run that stops at the first failure has then already executed
every other test.
"""
import numpy as np
import pytest
import torch

from tests.gpu_util import dev, ptr, stream

pytestmark = pytest.mark.gpu


def _inputs(nk, nv, seed):
    rng = np.random.default_rng(seed)
    f16 = np.float16
    C = (2 * nk + nv) * 128
    return C, dict(
        mixed=rng.standard_normal(C).astype(f16), z=rng.standard_normal(nv * 128).astype(f16),
        b=rng.standard_normal(nv).astype(f16), a=rng.standard_normal(nv).astype(f16),
        conv_w=(rng.standard_normal((C, 4)) * 0.5).astype(f16),
        conv_state=rng.standard_normal((C, 4)).astype(f16),
        A_log=np.log(rng.uniform(0.1, 16, nv)).astype(f16), dt_bias=np.ones(nv, dtype=f16),
        norm_w=(1 + 0.1 * rng.standard_normal(128)).astype(f16),
        state=(rng.standard_normal((nv, 128, 128)) * 0.1).astype(np.float32))


@pytest.mark.parametrize("nk,nv", [(16, 48), (2, 6)])
def test_noalloc_matches_regular_entry_point_twice(lib, nk, nv):
    C, x = _inputs(nk, nv, seed=nk + nv)
    ref = {k: dev(v) for k, v in x.items()}       # regular entry point, caller-provided scratch
    new = {k: dev(v) for k, v in x.items()}       # allocation-free entry point
    scratch = torch.zeros(C, dtype=torch.float32, device="cuda")
    out_ref = torch.zeros(nv * 128, dtype=torch.float16, device="cuda")
    out_new = torch.zeros(nv * 128, dtype=torch.float16, device="cuda")
    for call in range(2):
        mixed = np.random.default_rng(50 + call).standard_normal(C).astype(np.float16)
        for d in (ref, new):
            d["mixed"].copy_(torch.from_numpy(mixed))
        rc = lib.launch_dn_fused_heads(
            ptr(ref["mixed"]), ptr(ref["z"]), ptr(ref["b"]), ptr(ref["a"]), ptr(ref["conv_w"]),
            ptr(ref["conv_state"]), ptr(ref["A_log"]), ptr(ref["dt_bias"]), ptr(ref["norm_w"]),
            ptr(ref["state"]), ptr(scratch), ptr(out_ref), nk, nv, 1e-6, stream())
        assert rc == 0
        rc = lib.launch_dn_fused_noalloc(
            ptr(new["mixed"]), ptr(new["z"]), ptr(new["b"]), ptr(new["a"]), ptr(new["conv_w"]),
            ptr(new["conv_state"]), ptr(new["A_log"]), ptr(new["dt_bias"]), ptr(new["norm_w"]),
            ptr(new["state"]), ptr(out_new), nk, nv, 1e-6, stream())
        assert rc == 0
        torch.cuda.synchronize()
        assert np.isfinite(out_new.cpu().numpy().astype(np.float32)).all()
        # same kernels, same inputs: identical bytes (well inside the one-fp16-step tolerance the
        # other DeltaNet tests use)
        assert torch.equal(out_ref, out_new), f"call {call}: outputs differ"
        assert torch.equal(ref["state"], new["state"]), f"call {call}: recurrent state differs"
        assert torch.equal(ref["conv_state"], new["conv_state"]), f"call {call}: conv state differs"


def test_noalloc_rejects_oversized_shard(lib):
    import ctypes

    one = ctypes.c_void_p(0x1000)
    args = [one] * 11
    # 17 key + 51 value heads = 10880 channels > 10240: refused before any launch
    assert lib.launch_dn_fused_noalloc(*args, 17, 51, 1e-6, None) == -2
    assert lib.launch_dn_fused_noalloc(*args, 0, 3, 1e-6, None) == -1

"""Fused decode-step operators on the GPU, through the C ABI, against the CPU oracle.

The oracle returns the correctly rounded value of the reference's formula (fp16 rounding points
kept, float64 in between).  Tolerance: every fp16 output within ONE fp16 step of the oracle and at
least 99 % of outputs bit-identical; TWO steps where the formula rounds to fp16 twice in a row
(attention and DeltaNet outputs: an intermediate that lands on the other side of an fp16 boundary
moves the second rounding by up to two steps); fp32 state within 1e-5 of the state's scale.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import fused_ops_oracle as fo
from tests.gpu_util import dev, ptr, stream, ulp_diff_f16

pytestmark = pytest.mark.gpu


def assert_close_f16(got, want, min_exact=0.99, max_steps=1):
    d = ulp_diff_f16(got, want)
    assert d.max() <= max_steps, f"max fp16 step distance {d.max()}"
    assert (d == 0).mean() >= min_exact, (d == 0).mean()


@pytest.mark.parametrize("rows,n,stride", [(1, 5120, 5120), (24, 256, 512), (4, 256, 256),
                                           (3, 100, 128), (2, 2048, 2048), (1, 17408, 17408)])
def test_rmsnorm(lib, rows, n, stride):
    rng = np.random.default_rng(rows * n)
    buf = rng.standard_normal(rows * stride).astype(np.float16)
    w1 = (1.0 + rng.standard_normal(n) * 0.1).astype(np.float32)
    x = np.stack([buf[r * stride:r * stride + n] for r in range(rows)])
    want = fo.rmsnorm(x, w1, 1e-6)
    d_x, d_w = dev(buf), dev(w1)
    out = torch.zeros(rows * n, dtype=torch.float16, device="cuda")
    rc = lib.launch_rmsnorm(ptr(d_x), stride, ptr(d_w), ptr(out), rows, n, 1e-6, stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert_close_f16(out.cpu().numpy().reshape(rows, n), want)


def test_rmsnorm_unaligned_rows(lib):
    # a row view that starts 2 bytes off a 16-byte boundary takes the scalar path
    rng = np.random.default_rng(4)
    buf = rng.standard_normal(1 + 2 * 264).astype(np.float16)
    w1 = np.ones(256, dtype=np.float32)
    x = np.stack([buf[1 + r * 264:1 + r * 264 + 256] for r in range(2)])
    d_x, d_w = dev(buf), dev(w1)
    out = torch.zeros(2 * 256, dtype=torch.float16, device="cuda")
    rc = lib.launch_rmsnorm(ctypes.c_void_p(d_x.data_ptr() + 2), 264, ptr(d_w), ptr(out), 2, 256,
                            1e-6, stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert_close_f16(out.cpu().numpy().reshape(2, 256), fo.rmsnorm(x, w1, 1e-6))


def test_rope_qk_bit_exact(lib):
    rng = np.random.default_rng(8)
    q = rng.standard_normal((24, 256)).astype(np.float16)
    k = rng.standard_normal((4, 256)).astype(np.float16)
    pos = 575
    inv = 1.0 / (1e7 ** (np.arange(0, 256, 2) / 256.0))
    ang = np.concatenate([pos * inv, pos * inv])
    cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    d_q, d_k, d_c, d_s = dev(q), dev(k), dev(cos), dev(sin)
    qo, ko = torch.zeros_like(d_q), torch.zeros_like(d_k)
    rc = lib.launch_rope_qk(ptr(d_q), ptr(d_k), ptr(d_c), ptr(d_s), ptr(qo), ptr(ko), 24, 4,
                            stream())
    torch.cuda.synchronize()
    assert rc == 0
    # only products, sums and fp16 roundings of exact values: bit-exact
    assert np.array_equal(qo.cpu().numpy().view(np.uint16), fo.rope_qk(q, cos, sin).view(np.uint16))
    assert np.array_equal(ko.cpu().numpy().view(np.uint16), fo.rope_qk(k, cos, sin).view(np.uint16))


@pytest.mark.parametrize("n", [1, 255, 17408])
def test_silu_mul(lib, n):
    rng = np.random.default_rng(n)
    g = (rng.standard_normal(n) * 3).astype(np.float16)
    u = rng.standard_normal(n).astype(np.float16)
    d_g, d_u = dev(g), dev(u)
    out = torch.zeros(n, dtype=torch.float16, device="cuda")
    rc = lib.launch_silu_mul(ptr(d_g), ptr(d_u), ptr(out), n, stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert_close_f16(out.cpu().numpy(), fo.silu_mul(g, u))


def test_silu_mul_all_fp16_inputs(lib):
    # every finite fp16 gate value, u = 1: silu itself within one fp16 step everywhere
    bits = np.arange(0x10000, dtype=np.uint32).astype(np.uint16)
    g = bits.view(np.float16)
    g = g[np.isfinite(g)]
    u = np.ones_like(g)
    d_g, d_u = dev(g), dev(u)
    out = torch.zeros(len(g), dtype=torch.float16, device="cuda")
    rc = lib.launch_silu_mul(ptr(d_g), ptr(d_u), ptr(out), len(g), stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert_close_f16(out.cpu().numpy(), fo.silu_mul(g, u), min_exact=0.999)


@pytest.mark.parametrize("L,max_len", [(1, 64), (2, 64), (255, 1024), (256, 1024), (257, 1024),
                                       (575, 1024), (3072, 3072), (575, 3072), (1000, 20000)])
def test_attn_decode(lib, L, max_len):
    rng = np.random.default_rng(L + max_len)
    q = rng.standard_normal((24, 256)).astype(np.float16)
    gate = rng.standard_normal((24, 256)).astype(np.float16)
    keys = np.zeros((4, max_len, 256), dtype=np.float16)
    vals = np.zeros((4, max_len, 256), dtype=np.float16)
    keys[:, :L] = rng.standard_normal((4, L, 256)).astype(np.float16)
    vals[:, :L] = rng.standard_normal((4, L, 256)).astype(np.float16)
    # poison the unused tail: the kernel must not read past L
    keys[:, L:] = 12345.0
    vals[:, L:] = 12345.0
    scale = 256 ** -0.5
    want = fo.attn_decode(q, keys, vals, L, gate, scale)
    d = [dev(a) for a in (q, keys, vals, gate)]
    cum = torch.tensor([L], dtype=torch.int64, device="cuda")
    out = torch.zeros(24 * 256, dtype=torch.float16, device="cuda")
    rc = lib.launch_attn_decode(ptr(d[0]), ptr(d[1]), ptr(d[2]), ptr(cum), ptr(d[3]), ptr(out),
                                max_len, scale, stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert_close_f16(out.cpu().numpy().reshape(24, 256), want, min_exact=0.98, max_steps=2)


def make_dn_inputs(seed, state_scale=0.1):
    rng = np.random.default_rng(seed)
    f16 = np.float16
    return dict(
        mixed=rng.standard_normal(10240).astype(f16),
        z=rng.standard_normal(6144).astype(f16),
        b=rng.standard_normal(48).astype(f16),
        a=rng.standard_normal(48).astype(f16),
        conv_w=(rng.standard_normal((10240, 4)) * 0.5).astype(f16),
        conv_state=rng.standard_normal((10240, 4)).astype(f16),
        A_log=np.log(rng.uniform(0.1, 16, 48)).astype(f16),
        dt_bias=np.ones(48, dtype=f16),
        norm_w=(1 + 0.1 * rng.standard_normal(128)).astype(f16),
        state=(rng.standard_normal((48, 128, 128)) * state_scale).astype(np.float32),
    )


@pytest.mark.parametrize("seed", [0, 1])
def test_dn_fused_two_steps(lib, seed):
    x = make_dn_inputs(seed)
    d = {k: dev(v) for k, v in x.items()}
    scratch = torch.zeros(10240, dtype=torch.float32, device="cuda")
    out = torch.zeros(6144, dtype=torch.float16, device="cuda")
    conv_state, state = x["conv_state"], x["state"]
    for step in range(2):
        mixed = np.random.default_rng(100 + step + seed).standard_normal(10240).astype(np.float16)
        d["mixed"].copy_(torch.from_numpy(mixed))
        want_out, conv_state, state, want_scr = fo.dn_fused(
            mixed, x["z"], x["b"], x["a"], x["conv_w"], conv_state, x["A_log"], x["dt_bias"],
            x["norm_w"], state, 1e-6)
        rc = lib.launch_dn_fused(ptr(d["mixed"]), ptr(d["z"]), ptr(d["b"]), ptr(d["a"]),
                                 ptr(d["conv_w"]), ptr(d["conv_state"]), ptr(d["A_log"]),
                                 ptr(d["dt_bias"]), ptr(d["norm_w"]), ptr(d["state"]),
                                 ptr(scratch), ptr(out), 1e-6, stream())
        torch.cuda.synchronize()
        assert rc == 0
        # conv state is a pure shift: bit-exact
        assert np.array_equal(d["conv_state"].cpu().numpy().view(np.uint16),
                              conv_state.view(np.uint16))
        got_scr = scratch.cpu().numpy()
        assert_close_f16(got_scr.astype(np.float16), want_scr.astype(np.float16))
        got_state = d["state"].cpu().numpy()
        assert np.abs(got_state - state).max() <= 1e-5 * np.abs(state).max()
        assert_close_f16(out.cpu().numpy(), want_out, min_exact=0.97, max_steps=2)
        # carry the GPU's own state forward so one-step differences do not accumulate in the test
        state = got_state


@pytest.mark.parametrize("nk,nv", [(16, 48), (8, 24), (2, 6), (1, 3), (4, 4)])
def test_dn_fused_heads_shard(lib, nk, nv):
    # a tensor-parallel shard: fewer heads, same arithmetic
    rng = np.random.default_rng(nk * 100 + nv)
    f16 = np.float16
    C = (2 * nk + nv) * 128
    x = dict(
        mixed=rng.standard_normal(C).astype(f16), z=rng.standard_normal(nv * 128).astype(f16),
        b=rng.standard_normal(nv).astype(f16), a=rng.standard_normal(nv).astype(f16),
        conv_w=(rng.standard_normal((C, 4)) * 0.5).astype(f16),
        conv_state=rng.standard_normal((C, 4)).astype(f16),
        A_log=np.log(rng.uniform(0.1, 16, nv)).astype(f16), dt_bias=np.ones(nv, dtype=f16),
        norm_w=(1 + 0.1 * rng.standard_normal(128)).astype(f16),
        state=(rng.standard_normal((nv, 128, 128)) * 0.1).astype(np.float32))
    scr_want, conv_want = fo.dn_conv(x["mixed"], x["conv_w"], x["conv_state"])
    out_want, state_want = fo.dn_rec(scr_want, x["z"], x["b"], x["a"], x["A_log"], x["dt_bias"],
                                     x["norm_w"], x["state"], 1e-6, n_vheads=nv, n_kheads=nk)
    d = {k: dev(v) for k, v in x.items()}
    scratch = torch.zeros(C, dtype=torch.float32, device="cuda")
    out = torch.zeros(nv * 128, dtype=torch.float16, device="cuda")
    rc = lib.launch_dn_fused_heads(ptr(d["mixed"]), ptr(d["z"]), ptr(d["b"]), ptr(d["a"]),
                                   ptr(d["conv_w"]), ptr(d["conv_state"]), ptr(d["A_log"]),
                                   ptr(d["dt_bias"]), ptr(d["norm_w"]), ptr(d["state"]),
                                   ptr(scratch), ptr(out), nk, nv, 1e-6, stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(d["conv_state"].cpu().numpy().view(np.uint16), conv_want.view(np.uint16))
    assert np.abs(d["state"].cpu().numpy() - state_want).max() <= 1e-5 * np.abs(state_want).max()
    assert_close_f16(out.cpu().numpy(), out_want, min_exact=0.97, max_steps=2)


def test_dn_fused_heads_rejects_bad_counts(lib):
    one = ctypes.c_void_p(0x1000)
    args = [one] * 12
    assert lib.launch_dn_fused_heads(*args, 0, 3, 1e-6, None) == -1
    assert lib.launch_dn_fused_heads(*args, 4, 6, 1e-6, None) == -1


@pytest.mark.parametrize("hq,hkv,max_len", [(4, 2, 3072), (6, 1, 1024)])
def test_attn_decode_split_matches_single_cta_kernel(lib, hq, hkv, max_len):
    # keys split over eight CTAs per head, partial softmax results combined: same result as the
    # one-CTA kernel up to the last fp32 bit before the fp16 rounding; the head counters must be
    # back at zero after every call
    rng = np.random.default_rng(hq * 10 + hkv)
    keys = dev(rng.standard_normal((hkv, max_len, 256)).astype(np.float16))
    values = dev(rng.standard_normal((hkv, max_len, 256)).astype(np.float16))
    nbytes = lib.nvfp4_attn_split_scratch_bytes(hq)
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    scale = 256 ** -0.5
    for L in (1, 2, 15, 16, 17, 127, 128, 129, 575, 769, 1000, max_len):
        q = dev((rng.standard_normal(hq * 256) * 2).astype(np.float16))
        gate = dev(rng.standard_normal(hq * 256).astype(np.float16))
        ln = dev(np.array([L], dtype=np.int64))
        a = torch.zeros(hq * 256, dtype=torch.float16, device="cuda")
        b = torch.zeros_like(a)
        assert lib.launch_attn_decode_heads(ptr(q), ptr(keys), ptr(values), ptr(ln), ptr(gate),
                                            ptr(a), max_len, hq, hkv, scale, stream()) == 0
        assert lib.launch_attn_decode_split(ptr(q), ptr(keys), ptr(values), ptr(ln), ptr(gate),
                                            ptr(b), ptr(scratch), max_len, hq, hkv, scale,
                                            stream()) == 0
        torch.cuda.synchronize()
        steps = ulp_diff_f16(a.cpu().numpy(), b.cpu().numpy())
        # the fp16-rounded sum can move one step; the product with the rounded gate one more
        assert steps.max() <= 2 and (steps == 0).mean() > 0.98, (L, steps.max(), (steps == 0).mean())
        assert int(scratch[-4 * hq:].view(torch.int32).abs().sum()) == 0
    assert lib.launch_attn_decode_split(ptr(q), ptr(keys), ptr(values), ptr(ln), ptr(gate), ptr(b),
                                        None, max_len, hq, hkv, scale, stream()) == -2

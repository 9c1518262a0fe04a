"""Chunked prefill (tensor-core GEMM + chunk kernels) against the decode-step path.

Each chunk operator is checked against its decode twin or the CPU oracle on the same inputs; the
whole path is checked by prefilling a prompt and comparing caches, recurrent state and the greedy
continuation with feeding the prompt token by token through the decode step (which is itself
checked against the oracle model in tests/test_engine_gpu.py)."""
import numpy as np
import pytest
import torch

from oracle import fused_ops_oracle as fo
from tests.gpu_util import dev, ptr, stream, ulp_diff_f16

pytestmark = pytest.mark.gpu
SMALL = dict(hidden=256, inter=512, vocab=1000, n_layers=4, hq=2, hkv=1, dn_kheads=1,
             dn_vheads=2, max_len=64)
MARGIN = 4e-3


def test_transpose_and_residual_add(lib):
    rng = np.random.default_rng(0)
    for R, C, ld in ((5, 70, 8), (64, 64, 64), (13, 256, 16), (100, 33, 104)):
        a = rng.standard_normal((R, C)).astype(np.float16)
        d_a = dev(a)
        out = torch.full((C, ld), 7.0, dtype=torch.float16, device="cuda")
        assert lib.launch_transpose_f16(ptr(d_a), C, ptr(out), ld, R, C, stream()) == 0
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.array_equal(got[:, :R], a.T) and (got[:, R:] == 0).all(), (R, C)
    n, C, ldT = 13, 200, 16
    h = rng.standard_normal((n, C)).astype(np.float16)
    dT = rng.standard_normal((C, ldT)).astype(np.float16)
    d_h = dev(h)
    d_dT = dev(dT)
    assert lib.launch_add_transposed(ptr(d_h), ptr(d_dT), ldT, n, C, stream()) == 0
    torch.cuda.synchronize()
    want = (h.astype(np.float32) + dT[:, :n].T.astype(np.float32)).astype(np.float16)
    assert np.array_equal(d_h.cpu().numpy(), want)
    assert lib.launch_transpose_f16(None, 1, None, 1, 1, 1, None) == -1


def test_embed_rows_and_silu_mul_rows(lib):
    rng = np.random.default_rng(1)
    table = rng.standard_normal((50, 264)).astype(np.float16)
    ids = np.array([3, 49, 0, 3, 17], dtype=np.int64)
    out = torch.zeros((5, 264), dtype=torch.float16, device="cuda")
    d_table, d_ids = dev(table), dev(ids)
    assert lib.launch_embed_rows(ptr(d_table), ptr(d_ids), ptr(out), 5, 264, 50, stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), table[ids])

    inter, N = 24, 16
    g = rng.standard_normal((inter, N)).astype(np.float16) * 3
    u = rng.standard_normal((inter, N)).astype(np.float16)
    gu = np.empty((2 * inter, N), dtype=np.float16)            # interleave rows in groups of 8
    for j in range(inter // 8):
        gu[16 * j:16 * j + 8] = g[8 * j:8 * j + 8]
        gu[16 * j + 8:16 * j + 16] = u[8 * j:8 * j + 8]
    act = torch.zeros((inter, N), dtype=torch.float16, device="cuda")
    d_gu = dev(gu)
    assert lib.launch_silu_mul_rows(ptr(d_gu), ptr(act), inter, N, stream()) == 0
    torch.cuda.synchronize()
    want = fo.silu_mul(g.reshape(-1), u.reshape(-1)).reshape(inter, N)
    assert ulp_diff_f16(act.cpu().numpy(), want).max() <= 1


def test_attention_chunk_equals_token_by_token(lib):
    # same kernels' arithmetic per token: the chunk result must be bit-identical to running the
    # decode kernels once per token
    rng = np.random.default_rng(2)
    hq, hkv, max_len, n, p0 = 4, 2, 48, 9, 5
    ld = hq * 512 + 2 * hkv * 256
    qkv = rng.standard_normal((n, ld)).astype(np.float16)
    q_w1 = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    k_w1 = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    ang = rng.uniform(0, 6.28, (max_len, 256))
    cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    keys0 = rng.standard_normal((hkv, max_len, 256)).astype(np.float16)
    vals0 = rng.standard_normal((hkv, max_len, 256)).astype(np.float16)
    d = dict(qkv=dev(qkv), q_w1=dev(q_w1), k_w1=dev(k_w1), cos=dev(cos), sin=dev(sin))
    scale = 256 ** -0.5

    # token by token
    keys_a, vals_a = dev(keys0), dev(vals0)
    outs = []
    for t in range(n):
        pos = dev(np.array([p0 + t], dtype=np.int64))
        ln = dev(np.array([p0 + t + 1], dtype=np.int64))
        q = torch.zeros(hq * 256, dtype=torch.float16, device="cuda")
        g = torch.zeros_like(q)
        o = torch.zeros_like(q)
        assert lib.launch_attn_prep(ptr(d["qkv"][t]), ptr(d["q_w1"]), ptr(d["k_w1"]), ptr(d["cos"]),
                                    ptr(d["sin"]), ptr(pos), ptr(q), ptr(g), ptr(keys_a),
                                    ptr(vals_a), hq, hkv, max_len, 1e-6, stream()) == 0
        assert lib.launch_attn_decode_heads(ptr(q), ptr(keys_a), ptr(vals_a), ptr(ln), ptr(g),
                                            ptr(o), max_len, hq, hkv, scale, stream()) == 0
        torch.cuda.synchronize()
        outs.append(o.cpu().numpy())
    # one chunk
    keys_b, vals_b = dev(keys0), dev(vals0)
    q = torch.zeros((n, hq * 256), dtype=torch.float16, device="cuda")
    g = torch.zeros_like(q)
    o = torch.zeros_like(q)
    assert lib.launch_attn_prep_tokens(ptr(d["qkv"]), ld, ptr(d["q_w1"]), ptr(d["k_w1"]),
                                       ptr(d["cos"]), ptr(d["sin"]), p0, n, ptr(q), ptr(g),
                                       ptr(keys_b), ptr(vals_b), hq, hkv, max_len, 1e-6,
                                       stream()) == 0
    assert lib.launch_attn_prefill(ptr(q), ptr(keys_b), ptr(vals_b), p0 + 1, n, ptr(g), ptr(o),
                                   max_len, hq, hkv, scale, stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(keys_a, keys_b) and torch.equal(vals_a, vals_b)
    assert np.array_equal(o.cpu().numpy().view(np.uint16), np.stack(outs).view(np.uint16))
    assert lib.launch_attn_prefill(ptr(q), ptr(keys_b), ptr(vals_b), 0, n, ptr(g), ptr(o), max_len,
                                   hq, hkv, scale, stream()) == -2
    assert lib.launch_attn_prefill(ptr(q), ptr(keys_b), ptr(vals_b), max_len, n, ptr(g), ptr(o),
                                   max_len, hq, hkv, scale, stream()) == -2


@pytest.mark.parametrize("nk,nv,n", [(1, 2, 1), (2, 4, 3), (2, 6, 21)])
def test_deltanet_chunk_against_oracle_and_decode_kernel(lib, nk, nv, n):
    rng = np.random.default_rng(10 * nk + n)
    f16 = np.float16
    C = (2 * nk + nv) * 128
    ld = C + nv * 128 + 2 * nv
    ld += (-ld) % 4
    x = np.zeros((n, ld), dtype=f16)
    x[:, :C + nv * 128 + 2 * nv] = rng.standard_normal((n, C + nv * 128 + 2 * nv)).astype(f16)
    conv_w = (rng.standard_normal((C, 4)) * 0.5).astype(f16)
    conv_state = rng.standard_normal((C, 4)).astype(f16)
    A_log = np.log(rng.uniform(0.1, 16, nv)).astype(f16)
    dt_bias = np.ones(nv, dtype=f16)
    norm_w = (1 + 0.1 * rng.standard_normal(128)).astype(f16)
    state = (rng.standard_normal((nv, 128, 128)) * 0.1).astype(np.float32)

    # oracle, token by token
    cs, S = conv_state.copy(), state.copy()
    want = []
    for t in range(n):
        row = x[t]
        scr, cs = fo.dn_conv(row[:C], conv_w, cs)
        o, S = fo.dn_rec(scr, row[C:C + nv * 128], row[C + nv * 128:C + nv * 128 + nv],
                         row[C + nv * 128 + nv:C + nv * 128 + 2 * nv], A_log, dt_bias, norm_w, S,
                         1e-6, n_vheads=nv, n_kheads=nk)
        want.append(o)
    want = np.stack(want)

    d_cs, d_S = dev(conv_state), dev(state)
    d_x, d_w, d_A, d_dt, d_nw = dev(x), dev(conv_w), dev(A_log), dev(dt_bias), dev(norm_w)
    nbytes = lib.nvfp4_dn_prefill_work_bytes(n, nk, nv)
    work = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    out = torch.zeros((n, nv * 128), dtype=torch.float16, device="cuda")
    rc = lib.launch_dn_prefill(ptr(d_x), ld, ptr(d_w), ptr(d_cs), ptr(d_A), ptr(d_dt), ptr(d_nw),
                               ptr(d_S), ptr(work), nbytes, ptr(out), n, nk, nv, 1e-6, stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(d_cs.cpu().numpy().view(np.uint16), cs.view(np.uint16))
    # fp32 sums in another order than the oracle's; the difference accumulates over the tokens
    assert np.abs(d_S.cpu().numpy() - S).max() <= 1e-5 * (2 + n) * max(1.0, np.abs(S).max())
    steps = ulp_diff_f16(out.cpu().numpy(), want)
    assert steps.max() <= 4 and (steps <= 1).mean() > 0.97, (steps.max(), (steps <= 1).mean())
    # bad arguments
    assert lib.launch_dn_prefill(ptr(d_x), ld, ptr(d_w), ptr(d_cs), ptr(d_A), ptr(d_dt), ptr(d_nw),
                                 ptr(d_S), ptr(work), 16, ptr(out), n, nk, nv, 1e-6,
                                 stream()) == -1


def _engine(cfg, W):
    from nvfp4_v100_b200.engine import DecodeEngine

    eng = DecodeEngine(cfg, device="cuda")
    eng.load_weights(W)
    return eng


def _state(eng):
    n = int(eng.len.item())
    out = []
    for L in eng.layers:
        e = L.extra
        if L.attn:
            out.append(("kv", e["keys"][:, :n - 1].float().cpu().numpy(),
                        e["values"][:, :n - 1].float().cpu().numpy()))
        else:
            out.append(("dn", e["conv_state"].float().cpu().numpy(), e["state"].cpu().numpy()))
    return out


def test_engine_prefill_matches_token_by_token_and_oracle(lib):
    from nvfp4_v100_b200.engine import ModelConfig, rope_tables
    from oracle import decode_oracle as do

    cfg = ModelConfig(**SMALL)
    W = do.make_weights(cfg, 1)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, 14)
    n_gen = 12

    a = _engine(cfg, W)
    toks_a = a.run(prompt, n_gen)                       # teacher-forced prompt
    a.reset(int(prompt[0]))
    for t in range(1, len(prompt)):
        a.step()
        a.tok.fill_(int(prompt[t]))
    torch.cuda.synchronize()
    st_a = _state(a)

    b = _engine(cfg, W)
    b.reset(int(prompt[0]))
    b.prefill([int(t) for t in prompt[:-1]])            # one chunk
    assert int(b.pos.item()) == len(prompt) - 1 and int(b.len.item()) == len(prompt)
    st_b = _state(b)
    c = _engine(cfg, W)
    c.reset(int(prompt[0]))
    c.prefill([int(t) for t in prompt[:-1]], chunk=5)   # ragged chunks 5 + 5 + 3
    st_c = _state(c)

    def close(x, y, tol):
        scale = max(1e-3, float(np.abs(x).max()))
        return float(np.abs(x - y).max()) <= tol * scale

    for (ka, a1, a2), (_, b1, b2), (_, c1, c2) in zip(st_a, st_b, st_c):
        # GEMM vs GEMV: fp32 sums in another order, then the same fp16 roundings downstream
        assert close(a1, b1, 2e-2) and close(a2, b2, 2e-2), ka
        assert close(b1, c1, 2e-2) and close(b2, c2, 2e-2), ka

    toks_b = b.run(prompt, n_gen, native_prefill=True)
    cos, sin = rope_tables(cfg)
    want, _, margins = do.OracleModel(cfg, W, cos, sin).run(prompt, n_gen)
    for name, got in (("token-by-token", toks_a), ("prefill", toks_b)):
        for i in range(n_gen):
            if got[i] != want[i]:
                assert margins[i] < MARGIN, (name, i, got[i], want[i], margins[i])
                break
    assert toks_b[0] == want[0] or margins[0] < MARGIN

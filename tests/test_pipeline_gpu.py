"""The reference-style stack on the GPU: third-party model code + QLinear + patch_* + GraphDecoder
(nvfp4_v100_b200/pipeline/_qwen38_infer.py), checked the way the reference's acceptance scripts do
(pipeline/_qwen38_r1.py:269-296, experiments/_qwen38_p9_acc.py:90-119): greedy tokens of the fully
patched, graph-replayed stack against the unpatched eager stack from the same prefill state, in
one process.  A token may differ only where the eager stack's own top-1/top-2 margin is a few fp16
steps; the comparison stops there."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
tf = pytest.importorskip("transformers")
SMALL = dict(hidden=256, inter=512, vocab=1000, n_layers=4, hq=2, hkv=1, dn_kheads=1,
             dn_vheads=2, max_len=128, rope_theta=1e7)
MARGIN = 6e-3
N_GEN = 63          # the reference's acceptance length (pipeline/_qwen38_r1.py NDEC)


def compare_tokens(name, base, other, margins):
    """Token-for-token comparison with the baseline.  Equality over the whole length is required;
    the only escape is a step where the baseline's own top-1/top-2 logit margin is below MARGIN
    (a few fp16 steps): the two stacks may then legitimately pick different tokens, the
    comparison ends there and the margin is printed."""
    n = len(base) - 1
    matched, near_tie = 0, None
    for i in range(1, n + 1):
        if base[i] == other[i]:
            matched += 1
            continue
        assert margins[i - 1] < MARGIN, (name, i, base[i], other[i], margins[i - 1])
        near_tie = (i, margins[i - 1])
        break
    print(f"\n{name}: {matched}/{n} tokens identical to the baseline"
          + (f"; near-tie at step {near_tie[0]} (margin {near_tie[1]:.5f})" if near_tie else "")
          + f"; smallest margin {min(margins):.4f}")
    assert matched == n or near_tie is not None
    return matched


def write_container(tmp, cfg, W):
    from nvfp4_v100_b200.pipeline import _qwen38_nvfp4_pack as pk

    pre = "model.language_model."
    tensors, quant = {}, {}
    for name, val in W.items():
        if name == "embed_tokens":
            tensors[pre + "embed_tokens.weight"] = np.asarray(val, np.float16)
        elif name == "lm_head":
            quant["lm_head.weight"] = val
        elif isinstance(val, tuple):
            quant[pre + name + ".weight"] = val
        elif name == "norm.weight":
            tensors[pre + "norm.weight"] = np.asarray(val, np.float32)
        elif name.endswith("conv1d.weight"):
            tensors[pre + name] = np.asarray(val, np.float32).reshape(-1, 1, 4)
        else:
            tensors[pre + name] = np.asarray(val, np.float32)
    index = pk.pack_tensors(tensors, tmp, prequantised=quant)
    hf_cfg = dict(
        vocab_size=cfg.vocab, hidden_size=cfg.hidden, intermediate_size=cfg.inter,
        num_hidden_layers=cfg.n_layers, num_attention_heads=cfg.hq, num_key_value_heads=cfg.hkv,
        head_dim=256, linear_num_key_heads=cfg.dn_kheads, linear_num_value_heads=cfg.dn_vheads,
        linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4,
        rms_norm_eps=cfg.rms_eps, max_position_embeddings=cfg.max_len, tie_word_embeddings=False,
        rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta,
                         "partial_rotary_factor": 1.0})
    json.dump(hf_cfg, open(os.path.join(tmp, "config.json"), "w"))
    return index


def snap_all(model, cache, L, Q):
    kv = Q.snap_decode_state(model, cache, L)
    lin = []
    for i, lay in enumerate(cache.layers):
        if hasattr(lay, "conv_states"):
            lin.append((i, lay.conv_states.clone(), lay.recurrent_states.clone()))
    return kv, lin


def restore_all(model, cache, snap, L, Q):
    kv, lin = snap
    Q.restore_decode_state(model, cache, kv, L)
    for i, c, r in lin:
        cache.layers[i].conv_states.copy_(c)
        cache.layers[i].recurrent_states.copy_(r)


def test_patched_graph_stack_matches_eager_stack(lib, tmp_path):
    from transformers import StaticCache

    from nvfp4_v100_b200.engine import ModelConfig
    from nvfp4_v100_b200.pipeline import _qwen38_infer as Q
    from oracle import decode_oracle as do

    cfg = ModelConfig(**SMALL)
    W = do.make_weights(cfg, 1)
    index = write_container(str(tmp_path), cfg, W)
    assert index["lm_head.weight"]["fmt"] == "nvfp4_v2_embedded_sign"
    hf_cfg, model = Q.build_model(str(tmp_path))
    assert isinstance(model.lm_head, Q.QLinear) and model.lm_head.M == cfg.vocab

    prompt = np.random.default_rng(1).integers(0, cfg.vocab, 8)
    ids = torch.from_numpy(prompt).cuda().view(1, -1)
    L, n_gen = ids.shape[1], N_GEN

    # ---- stack 0: baseline, eager with a growing (dynamic) cache ----
    from transformers import DynamicCache

    dyn = DynamicCache(config=model.config)
    with torch.no_grad():
        out0 = model(ids, past_key_values=dyn, use_cache=True)
        cur = int(out0.logits[0, -1].float().argmax())
        toks_0, margins = [cur], []
        for t in range(n_gen):
            o = model(torch.tensor([[cur]], device="cuda"), past_key_values=dyn, use_cache=True,
                      cache_position=torch.tensor([L + t], device="cuda"))
            lg = o.logits[0, -1].float()
            top2 = torch.topk(lg, 2).values
            margins.append(float(top2[0] - top2[1]))
            cur = int(lg.argmax())
            toks_0.append(cur)
    del dyn

    cache = StaticCache(config=model.config, max_cache_len=cfg.max_len)
    first = Q.prefill(model, cache, ids)              # T = 8: every QLinear takes the GEMM path
    assert first == toks_0[0]
    snap = snap_all(model, cache, L, Q)
    emb_w = model.model.embed_tokens.weight_cpu

    # ---- stack A: eager, static cache, unpatched (third-party operators + QLinear GEMV) ----
    toks_a = [first]
    cur = first
    with torch.no_grad():
        for t in range(n_gen):
            o = model(torch.tensor([[cur]], device="cuda"), past_key_values=cache, use_cache=True,
                      cache_position=torch.tensor([L + t], device="cuda"))
            cur = int(o.logits[0, -1].float().argmax())
            toks_a.append(cur)

    # ---- stack G: the unpatched step in a CUDA graph (static cache) ----
    restore_all(model, cache, snap, L, Q)
    dec_g = Q.GraphDecoder(model, cache, L, cfg.hidden)
    restore_all(model, cache, snap, L, Q)
    dec_g.reset_pos()
    torch.cuda.synchronize()
    toks_g = [first]
    cur = first
    with torch.no_grad():
        for _ in range(n_gen):
            cur = dec_g.step(cur, emb_w)
            toks_g.append(cur)
    del dec_g

    # ---- stack B: every fused kernel + the whole step in a CUDA graph ----
    restore_all(model, cache, snap, L, Q)
    mods = Q.patch_fused_deltanet(model, cache)
    Q.patch_attn_decode(model, cache, max_len=cfg.max_len)
    Q.patch_rmsnorm(model)
    Q.patch_rope()
    Q.patch_mlp_silu_mul(model)
    vf_snap = [(m._vf_conv.clone(), m._vf_S.clone()) for m in mods]
    dec = Q.GraphDecoder(model, cache, L, cfg.hidden)
    restore_all(model, cache, snap, L, Q)             # warm-up and capture advanced the state
    for m, (c, s) in zip(mods, vf_snap):
        m._vf_conv.copy_(c)
        m._vf_S.copy_(s)
    dec.reset_pos()
    torch.cuda.synchronize()
    toks_b = [first]
    cur = first
    with torch.no_grad():
        for _ in range(n_gen):
            cur = dec.step(cur, emb_w)
            toks_b.append(cur)

    # ---- two tokens per replay (speculative verify): positions [p, p + 1] from the same state ----
    restore_all(model, cache, snap, L, Q)
    for m, (c, s) in zip(mods, vf_snap):
        m._vf_conv.copy_(c)
        m._vf_S.copy_(s)
    pos2 = torch.tensor([L, L + 1], device="cuda")
    dec2 = Q.GraphDecoder2(model, cache, L, cfg.hidden, pos2, n_warmup=1)
    restore_all(model, cache, snap, L, Q)
    for m, (c, s) in zip(mods, vf_snap):
        m._vf_conv.copy_(c)
        m._vf_S.copy_(s)
    pos2.copy_(torch.tensor([L, L + 1]))
    torch.cuda.synchronize()
    nxt2, lg2 = dec2.step2(toks_b[0], toks_b[1], emb_w)
    nxt2 = nxt2.cpu().tolist()
    # after tokA the model must predict what the one-token decoder predicted (tokB), and after
    # tokB the decoder's third token, unless the eager margin there is a near-tie
    for got, want_tok, margin in ((nxt2[0], toks_b[1], margins[0]), (nxt2[1], toks_b[2], margins[1])):
        assert got == want_tok or margin < MARGIN, (nxt2, toks_b[:3], margins[:2])
    assert torch.isfinite(lg2.float()).all() and pos2.cpu().tolist() == [L + 1, L + 2]

    # the reference's matrix (pipeline/_qwen38_r1.py:241-296): dynamic cache, static cache eager,
    # static cache + graph, graph + fused kernels - 63 tokens each, against the first
    compare_tokens("eager, static cache", toks_0, toks_a, margins)
    compare_tokens("graph, static cache", toks_0, toks_g, margins)
    compare_tokens("graph + fused kernels", toks_0, toks_b, margins)
    # restore the module-level patch for other tests in this process
    from transformers.models.qwen3_5 import modeling_qwen3_5 as hf
    hf.apply_rotary_pos_emb = hf._vf_rope_orig


def test_qlinear_dispatch_by_token_count(lib):
    from nvfp4_v100_b200.pipeline import _qwen38_infer as Q
    from oracle import nvfp4_codec_oracle as oc

    M, K = 320, 512
    w = oc.synthetic_weight(M, K, seed=2)
    p, s = oc.encode(w)
    d_p, d_s = torch.from_numpy(p).cuda(), torch.from_numpy(s).cuda()
    lin = Q.QLinear(d_p.data_ptr(), d_s.data_ptr(), M, K)
    wd = oc.decode_f64(p, s)
    for T in (1, 2, 3, 8, 40):
        x = torch.randn(1, T, K, device="cuda").half()
        y = lin(x)
        assert y.shape == (1, T, M)
        ref = x[0].double().cpu().numpy() @ wd.T
        assert oc.rel_error_floored(y[0].cpu().numpy(), ref).max() <= 2e-3, T


def test_qlinear_keeps_ragged_token_counts_on_the_tensor_cores(lib):
    # 13 tokens (a ragged last prefill chunk): the bridge hands its [tokens, K] rows to the
    # token-major GEMM entry, which takes any token count on the tensor-core kernel; the result
    # equals the oracle's, and equals the same rows of a 16-token call bit for bit.  A K that the
    # tensor-core kernel does not take (112) goes through the reference-shaped padded call.
    from nvfp4_v100_b200.pipeline import _qwen38_infer as Q
    from oracle import nvfp4_codec_oracle as oc

    M, K = 384, 1024
    w = oc.synthetic_weight(M, K, seed=4)
    p, s = oc.encode(w)
    d_p, d_s = torch.from_numpy(p).cuda(), torch.from_numpy(s).cuda()
    lin = Q.QLinear(d_p.data_ptr(), d_s.data_ptr(), M, K)
    wd = oc.decode_f64(p, s)
    lib.nvfp4_gemm_status(1)
    x16 = torch.randn(1, 16, K, device="cuda").half()
    y16 = lin(x16)
    for T in (13, 3, 7, 511):
        x = x16[:, :T] if T <= 16 else torch.randn(1, T, K, device="cuda").half()
        y = lin(x)
        assert y.shape == (1, T, M)
        ref = x[0].double().cpu().numpy() @ wd.T
        assert oc.rel_error_floored(y[0].cpu().numpy(), ref).max() <= 2e-3, T
        if T <= 16:
            assert torch.equal(y, y16[:, :T]), T      # same kernel, same tile, same arithmetic
    assert lib.nvfp4_gemm_status(0) == 0
    M2, K2 = 100, 112
    p2, s2 = oc.encode(oc.synthetic_weight(M2, K2, seed=5))
    d_p2, d_s2 = torch.from_numpy(p2).cuda(), torch.from_numpy(s2).cuda()
    lin2 = Q.QLinear(d_p2.data_ptr(), d_s2.data_ptr(), M2, K2)
    x = torch.randn(1, 13, K2, device="cuda").half()
    ref = x[0].double().cpu().numpy() @ oc.decode_f64(p2, s2).T
    assert oc.rel_error_floored(lin2(x)[0].cpu().numpy(), ref).max() <= 2e-3


def test_pair_fusion_of_small_projections(lib):
    # experiments/_qwen38_p7_pair.py: (in_proj_b, in_proj_a) and (k_proj, v_proj) share one launch;
    # rows are independent, so the members' outputs are bit-identical to separate launches
    import torch.nn as nn

    from nvfp4_v100_b200.experiments import _qwen38_p7_pair as P7
    from nvfp4_v100_b200.pipeline import _qwen38_infer as Q
    from oracle import nvfp4_codec_oracle as oc

    K = 512

    def qlin(M, seed):
        w = oc.synthetic_weight(M, K, seed=seed)
        p, s = oc.encode(w)
        d_p, d_s = Q.GEMV.gpu_malloc(p.nbytes), Q.GEMV.gpu_malloc(s.nbytes)
        assert Q.GEMV.gpu_memcpy_h2d(d_p, p.ctypes.data, p.nbytes) == 0
        assert Q.GEMV.gpu_memcpy_h2d(d_s, s.ctypes.data, s.nbytes) == 0
        return Q.QLinear(d_p, d_s, M, K), (p, s)

    class Block(nn.Module):
        pass

    model = nn.Module()
    model.linear_attn = Block()
    model.self_attn = Block()
    raw = {}
    for owner, names, M in ((model.linear_attn, ("in_proj_b", "in_proj_a"), 48),
                            (model.self_attn, ("k_proj", "v_proj"), 256)):
        for i, n in enumerate(names):
            lin, raw[n] = qlin(M, seed=len(raw) + 1)
            setattr(owner, n, lin)
    x = torch.randn(1, 1, K, device="cuda").half()
    before = {n: getattr(o, n)(x).clone() for o, ns in ((model.linear_attn, ("in_proj_b", "in_proj_a")),
                                                        (model.self_attn, ("k_proj", "v_proj")))
              for n in ns}
    assert P7.patch_pair_gemv(model) == 2
    for owner, lead, follower in ((model.linear_attn, "in_proj_b", "in_proj_a"),
                                  (model.self_attn, "k_proj", "v_proj")):
        a, b = getattr(owner, lead), getattr(owner, follower)
        assert isinstance(a, P7._PairLinear) and isinstance(b, P7._PairLinear) and a._group is b._group
        ya = a(x)            # the lead launches the whole group
        yb = b(x)            # the follower takes its rows from that launch
        assert torch.equal(ya, before[lead]) and torch.equal(yb, before[follower])
        # unexpected order or several tokens: every member still works on its own rows
        x3 = torch.randn(1, 3, K, device="cuda").half()
        ref = x3[0].double().cpu().numpy() @ oc.decode_f64(*raw[follower]).T
        assert oc.rel_error_floored(b(x3)[0].cpu().numpy(), ref).max() <= 2e-3
        other = torch.randn(1, 1, K, device="cuda").half()
        ref1 = other[0].double().cpu().numpy() @ oc.decode_f64(*raw[follower]).T
        assert oc.rel_error_floored(b(other)[0].cpu().numpy(), ref1).max() <= 1e-3

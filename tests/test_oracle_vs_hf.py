"""Second opinion for the CPU oracle model: the third-party model code the reference wraps
(transformers Qwen3_5ForCausalLM, the version installed here) run in fp32 on CPU with the same
dequantised weights.  It pins the SEMANTICS of the decode step — per-head [q | gate] layout of
q_proj, zero-centred RMSNorm, full-rotation RoPE, the conv window, the gated delta rule with its
state orientation, the gated RMSNorm, residual structure — independently of this repository's
kernels.  Numerics differ (fp32 everywhere there, fp16 rounding points here), so logits are
compared with a tolerance and tokens where the margin is clear."""
import numpy as np
import pytest
import torch

from nvfp4_v100_b200.engine import ModelConfig, rope_tables
from oracle import decode_oracle as do
from oracle import nvfp4_codec_oracle as oc

tf = pytest.importorskip("transformers")

SMALL = dict(hidden=256, inter=512, vocab=300, n_layers=4, hq=2, hkv=1, dn_kheads=1,
             dn_vheads=2, max_len=32, rope_theta=1e7)


def build_hf(cfg: ModelConfig, W):
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM

    hf_cfg = Qwen3_5TextConfig(
        vocab_size=cfg.vocab, hidden_size=cfg.hidden, intermediate_size=cfg.inter,
        num_hidden_layers=cfg.n_layers, num_attention_heads=cfg.hq, num_key_value_heads=cfg.hkv,
        head_dim=256, linear_num_key_heads=cfg.dn_kheads, linear_num_value_heads=cfg.dn_vheads,
        linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4,
        rms_norm_eps=cfg.rms_eps, max_position_embeddings=cfg.max_len, tie_word_embeddings=False,
        rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta,
                         "partial_rotary_factor": 1.0})
    assert list(hf_cfg.layer_types) == ["full_attention" if cfg.is_attn(i) else "linear_attention"
                                        for i in range(cfg.n_layers)]
    model = Qwen3_5ForCausalLM(hf_cfg).eval().float()
    sd = {}
    for name, val in W.items():
        if isinstance(val, tuple):
            t = torch.from_numpy(oc.decode_f64(*val).astype(np.float32))
        else:
            t = torch.from_numpy(np.asarray(val, dtype=np.float32))
        if name == "embed_tokens":
            key = "model.embed_tokens.weight"
        elif name == "norm.weight":
            key = "model.norm.weight"
        elif name == "lm_head":
            key = "lm_head.weight"
        else:
            key = "model." + name
            if isinstance(val, tuple):
                key += ".weight"
            if key.endswith("conv1d.weight"):
                t = t.reshape(-1, 1, 4)
        sd[key] = t
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in m or "inv_freq" in m for m in missing), missing
    return model, hf_cfg


def test_oracle_step_matches_hf_model():
    from transformers import DynamicCache

    cfg = ModelConfig(**SMALL)
    W = do.make_weights(cfg, 3)
    cos, sin = rope_tables(cfg)
    oracle = do.OracleModel(cfg, W, cos, sin)
    model, hf_cfg = build_hf(cfg, W)
    prompt = [5, 77, 123, 9, 250, 31]
    cache = DynamicCache(config=hf_cfg)
    worst = 0.0
    agree = 0
    with torch.no_grad():
        for t, tok in enumerate(prompt + [0] * 6):
            if t >= len(prompt):
                tok = nxt                                   # greedy continuation of the HF model
            want = model(torch.tensor([[tok]]), past_key_values=cache, use_cache=True).logits[0, -1]
            got = oracle.step(int(tok)).astype(np.float32)
            w = want.numpy()
            err = np.abs(got - w).max() / np.abs(w).max()
            worst = max(worst, err)
            nxt = int(w.argmax())
            top2 = np.sort(w)[-2:]
            if top2[1] - top2[0] > 0.02 * np.abs(w).max():
                assert int(got.argmax()) == nxt, (t, err)
                agree += 1
    # fp16 rounding points on one side, fp32 on the other
    assert worst < 3e-2, worst
    assert agree >= 3

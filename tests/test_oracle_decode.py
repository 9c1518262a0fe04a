"""The CPU oracle model: deterministic, shape-consistent, and built from the pinned blocks."""
import numpy as np

from nvfp4_v100_b200.engine import ModelConfig, rope_tables
from oracle import decode_oracle as do

SMALL = dict(hidden=256, inter=512, vocab=300, n_layers=4, hq=2, hkv=1, dn_kheads=1,
             dn_vheads=2, max_len=32)


def test_oracle_model_runs_and_is_deterministic():
    cfg = ModelConfig(**SMALL)
    cos, sin = rope_tables(cfg)
    W = do.make_weights(cfg, 0)
    a = do.OracleModel(cfg, W, cos, sin).run([1, 2, 3], 5)
    b = do.OracleModel(cfg, do.make_weights(cfg, 0), cos, sin).run([1, 2, 3], 5)
    assert a[0] == b[0] and len(a[0]) == 5
    assert all(l.shape == (cfg.vocab,) and l.dtype == np.float16 for l in a[1])
    assert np.isfinite(np.stack(a[1]).astype(np.float32)).all()


def test_layer_pattern_and_shapes():
    cfg = ModelConfig()
    kinds = [cfg.is_attn(i) for i in range(cfg.n_layers)]
    assert sum(kinds) == 16 and kinds[3] and not kinds[0]
    n = 0
    total = 0
    for i in range(cfg.n_layers):
        for M, K in cfg.layer_shapes(i).values():
            n += 1
            total += M * K
    n += 1
    total += cfg.vocab * cfg.hidden
    assert n == 497                       # the reference's per-step GEMV count
    assert total == 25_621_954_560        # weights per step


def test_rope_table_matches_definition():
    cfg = ModelConfig(max_len=8)
    cos, sin = rope_tables(cfg)
    assert cos.shape == (8, 256) and cos.dtype == np.float16
    assert np.all(cos[0] == 1) and np.all(sin[0] == 0)
    assert np.array_equal(cos[:, :128], cos[:, 128:])
    assert abs(float(sin[1, 0]) - np.sin(1.0)) < 1e-3

"""The container -> tensor-parallel shard path on the CPU: a reference-format container is
written from the oracle's weights, mapped, and every rank's shard taken from the map must be the
same bytes as the shard cut from the in-memory arrays; reading a shard must touch only views of
the map until the final copy."""
import numpy as np
import pytest

from nvfp4_v100_b200 import tp
from oracle import decode_oracle as do

SMALL = dict(hidden=256, inter=512, vocab=1000, n_layers=4, hq=4, hkv=2, dn_kheads=2, dn_vheads=4,
             max_len=64)


def write_container(tmp, W):
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
        elif name.endswith("conv1d.weight"):
            tensors[pre + name] = np.asarray(val, np.float32).reshape(-1, 1, 4)
        else:
            tensors[pre + name] = np.asarray(val, np.float32)
    return pk.pack_tensors(tensors, tmp, prequantised=quant)


def test_container_views_and_shards_equal_the_in_memory_weights(tmp_path):
    # importing the engine module needs torch but no GPU
    from nvfp4_v100_b200.engine import ContainerWeights, ModelConfig

    cfg = ModelConfig(**SMALL)
    W = do.make_weights(cfg, 3)
    write_container(str(tmp_path), W)
    C = ContainerWeights(str(tmp_path))
    for name, val in W.items():
        got = C[name]
        if isinstance(val, tuple):
            assert isinstance(got[0], np.memmap) or isinstance(got[0].base, (np.memmap, np.ndarray))
            assert np.array_equal(got[0], val[0]) and np.array_equal(got[1], val[1]), name
        else:
            assert np.array_equal(np.asarray(got, np.float16).reshape(np.asarray(val).shape),
                                  np.asarray(val, np.float16)), name
    with pytest.raises(KeyError):
        C["layers.0.no_such_weight"]
    # per-rank shards: rows for column-parallel layers, a strided K range for row-parallel ones
    for world in (2, 4):
        for rank in range(world):
            p, s = C["layers.3.self_attn.q_proj"]
            lo, hi = tp.split_range(p.shape[0], world, rank, 512)
            a = tp.shard_rows(p, s, lo, hi)
            b = tp.shard_rows(*W["layers.3.self_attn.q_proj"], lo, hi)
            assert a[0].base is not None              # still a view of the map: nothing copied yet
            assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
            p, s = C["layers.0.mlp.down_proj"]
            pk, sk, k0, k1 = tp.shard_k(p, s, cfg.inter, world, rank)
            wk = tp.shard_k(*W["layers.0.mlp.down_proj"], cfg.inter, world, rank)
            assert (k0, k1) == (wk[2], wk[3]) and not pk.flags["C_CONTIGUOUS"]
            assert np.array_equal(np.ascontiguousarray(pk), wk[0])
            assert np.array_equal(np.ascontiguousarray(sk), wk[1])
            assert np.ascontiguousarray(pk).nbytes == p.nbytes // world   # shard-sized host copy

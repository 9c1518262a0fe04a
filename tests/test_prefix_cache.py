"""Prefix-state cache: LRU bookkeeping on the CPU with a stand-in engine, and on the GPU that a
prompt continued from a cached prefix generates exactly what a full prefill generates
(reference behaviour: experiments/_qwen38_p4a_lru.py:210-246 — byte-capped LRU, hit / miss / evict
counters, poisoned state between requests)."""
import numpy as np
import pytest
import torch

from nvfp4_v100_b200.prefix_cache import PrefixCache, generate, snapshot_bytes


class FakeEngine:
    def __init__(self):
        self.state = torch.zeros(256, dtype=torch.float32)      # 1 KiB per snapshot

    def snapshot(self):
        return {"s": self.state.clone(), "layers": [(self.state[:0].clone(),)]}

    def restore(self, snap):
        self.state.copy_(snap["s"])


def test_lru_order_budget_and_longest_prefix():
    eng = FakeEngine()
    cache = PrefixCache(eng, max_bytes=3 * 1024)
    base = list(range(100, 140))
    for n in (8, 16, 24):
        eng.state.fill_(float(n))
        cache.put(base[:n])
    assert cache.bytes_used == 3 * 1024 == sum(snapshot_bytes(e[1]) for e in cache.store.values())
    # longest proper prefix wins and refreshes its entry
    eng.state.fill_(-1.0)
    assert cache.get(base[:30]) == 24 and float(eng.state[0]) == 24.0
    assert cache.get(base[:20]) == 16 and float(eng.state[0]) == 16.0
    # an exact-length prompt must leave one token to process: the 16-token entry is not used
    assert cache.get(base[:16]) == 8
    # a prompt that diverges inside the shortest prefix misses and leaves the engine alone
    eng.state.fill_(-2.0)
    other = [7] + base[1:30]
    assert cache.get(other) == 0 and float(eng.state[0]) == -2.0
    assert (cache.hit, cache.miss, cache.evict) == (3, 1, 0)
    # a fourth entry evicts the least recently used one (24: 8 and 16 were touched after it)
    eng.state.fill_(32.0)
    cache.put(base[:32])
    assert cache.evict == 1 and cache.key_of(base[:24]) not in cache.store
    assert cache.get(base[:40]) == 32
    # the newest entry survives even a budget smaller than one snapshot
    tiny = PrefixCache(eng, max_bytes=10)
    tiny.put(base[:4])
    tiny.put(base[:6])
    assert len(tiny.store) == 1 and tiny.evict == 1 and tiny.get(base[:10]) == 6
    # re-putting a key replaces it without double counting
    cache.put(base[:32])
    assert cache.bytes_used == len(cache.store) * 1024


@pytest.mark.gpu
def test_generation_from_cached_prefix_equals_full_prefill(lib):
    from nvfp4_v100_b200.engine import DecodeEngine, ModelConfig
    from oracle import decode_oracle as do

    cfg = ModelConfig(hidden=256, inter=512, vocab=1000, n_layers=4, hq=2, hkv=1, dn_kheads=1,
                      dn_vheads=2, max_len=64)
    W = do.make_weights(cfg, 1)
    eng = DecodeEngine(cfg, device="cuda")
    eng.load_weights(W)
    eng.reset(0)
    eng.capture(n_warmup=1)
    rng = np.random.default_rng(3)
    shared = rng.integers(0, cfg.vocab, 20)
    p1 = np.concatenate([shared, rng.integers(0, cfg.vocab, 7)])
    p2 = np.concatenate([shared, rng.integers(0, cfg.vocab, 11)])
    n_gen = 10
    full1 = eng.run(p1, n_gen, native_prefill=True)
    full2 = eng.run(p2, n_gen, native_prefill=True)

    cache = PrefixCache(eng, max_bytes=64 << 20)
    got1, reused1 = generate(eng, cache, p1, n_gen, remember=len(shared))
    assert reused1 == 0 and cache.miss == 1 and len(cache.store) == 1
    # poison everything a request leaves behind, as the reference's test does between requests
    for L in eng.layers:
        for name in ("keys", "values", "conv_state", "state"):
            if name in L.extra:
                L.extra[name].fill_(12345.0)
    got2, reused2 = generate(eng, cache, p2, n_gen)
    assert reused2 == len(shared) and cache.hit == 1
    assert got1 == full1 and got2 == full2
    assert eng.lib.nvfp4_gemm_status(0) == 0

"""Prefix-state cache: snapshots of a sequence's decode state (KV prefix of every attention
layer, conv window and recurrent state of every DeltaNet layer, counters) kept under a byte
budget with least-recently-used eviction, so that a prompt that starts with a cached prefix only
prefills the remainder.

The reference keeps such snapshots in host RAM because its 16 GB V100 has no room for them
(experiments/_qwen38_p4a_lru.py:210-246: exact-key lookup, byte-capped ``OrderedDict``, hit / miss /
evict counters, at least one entry always kept).  Here the snapshots stay in device memory — a
512-token prefix of the 27B model is 67 MB of KV + 151 MB of DeltaNet state, and a B200 has 180 GB —
so a hit costs device-to-device copies only.  Lookup returns the LONGEST cached prefix of the
prompt, not only an exact match.

The cache works with any object that has ``snapshot()`` / ``restore(snapshot)`` where a snapshot
is a (nested) structure of tensors — ``DecodeEngine`` in this package.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict

import numpy as np


def _tensors(obj):
    if hasattr(obj, "numel") and hasattr(obj, "element_size"):
        yield obj
    elif isinstance(obj, dict):
        for v in obj.values():
            yield from _tensors(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _tensors(v)


def snapshot_bytes(snap) -> int:
    return sum(t.numel() * t.element_size() for t in _tensors(snap))


class PrefixCache:
    def __init__(self, engine, max_bytes: int):
        self.engine = engine
        self.max_bytes = int(max_bytes)
        self.store: OrderedDict[str, tuple] = OrderedDict()   # key -> (n_tokens, snapshot, bytes)
        self.lengths: dict[int, int] = {}                     # prefix length -> entries of it
        self.hit = self.miss = self.evict = 0

    @staticmethod
    def key_of(tokens) -> str:
        ids = np.ascontiguousarray(np.asarray(tokens, dtype=np.int64))
        return hashlib.sha256(ids.tobytes()).hexdigest()[:16]

    @property
    def bytes_used(self) -> int:
        return sum(e[2] for e in self.store.values())

    def put(self, tokens) -> str:
        """Remember the engine's CURRENT state as the state after ``tokens``.  Evicts the least
        recently used entries until the budget holds (the newest entry always stays)."""
        key = self.key_of(tokens)
        if key in self.store:
            self._forget(key)
        snap = self.engine.snapshot()
        self.store[key] = (len(tokens), snap, snapshot_bytes(snap))
        self.lengths[len(tokens)] = self.lengths.get(len(tokens), 0) + 1
        while len(self.store) > 1 and self.bytes_used > self.max_bytes:
            victim = next(iter(self.store))
            self._forget(victim)
            self.evict += 1
        return key

    def _forget(self, key: str) -> None:
        n, _, _ = self.store.pop(key)
        self.lengths[n] -= 1
        if not self.lengths[n]:
            del self.lengths[n]

    def get(self, prompt) -> int:
        """Restore the engine to the longest cached prefix of ``prompt`` and return its length
        (0 and an untouched engine on a miss).  Only proper prefixes that leave at least one
        token to process are considered."""
        prompt = np.asarray(prompt, dtype=np.int64)
        for n in sorted(self.lengths, reverse=True):
            if n >= len(prompt):
                continue
            key = self.key_of(prompt[:n])
            entry = self.store.get(key)
            if entry is not None:
                self.store.move_to_end(key)
                self.engine.restore(entry[1])
                self.hit += 1
                return n
        self.miss += 1
        return 0


def generate(engine, cache: PrefixCache, prompt, n_gen: int, remember: int = 0):
    """Greedy generation with prefix reuse on a ``DecodeEngine``: restore the longest cached
    prefix, prefill what is left of the prompt (all but its last token, which goes through the
    decode step), optionally remember the state after the first ``remember`` prompt tokens, and
    generate ``n_gen`` tokens.  Returns (tokens, length of the reused prefix)."""
    import torch

    prompt = [int(t) for t in prompt]
    engine.reset(prompt[0])
    reused = cache.get(prompt)
    body_end = len(prompt) - 1                       # tokens [reused, body_end) still to prefill
    if remember and reused < remember <= body_end:
        engine.prefill(prompt[reused:remember], start=reused)
        cache.put(prompt[:remember])
        reused_to = remember
    else:
        reused_to = reused
    if body_end > reused_to:
        engine.prefill(prompt[reused_to:body_end], start=reused_to)
    engine.pos.fill_(body_end)
    engine.len.fill_(body_end + 1)
    engine.tok.fill_(prompt[-1])
    engine.hist_count.zero_()
    for _ in range(n_gen):
        engine.step()
    torch.cuda.synchronize()
    return engine.history[:n_gen].cpu().tolist(), reused

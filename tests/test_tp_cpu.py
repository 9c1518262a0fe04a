"""Tensor-parallel sharding logic on CPU: two gloo ranks compute their shards of a column-split
and a K-split NVFP4 layer with the oracle, exchange results with the real collectives, and must
reproduce the unsharded oracle result."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nvfp4_v100_b200 import tp
from oracle import nvfp4_codec_oracle as oc


def test_split_range_covers_everything():
    for n, unit in ((5120, 128), (17408, 128), (48, 1), (24, 1), (6144, 128)):
        for world in (1, 2, 4, 8):
            got = [tp.split_range(n, world, r, unit) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            assert all((hi - lo) % unit == 0 for lo, hi in got)


def test_kv_heads_replicated_when_more_ranks_than_heads():
    p = np.arange(4 * 256 * 8, dtype=np.uint8).reshape(4 * 256, 8)
    s = np.zeros((4 * 256, 1), dtype=np.uint8)
    heads = [tp.shard_kv_heads(p, s, 4, 8, r)[2:] for r in range(8)]
    assert heads == [(0, 1), (0, 1), (1, 2), (1, 2), (2, 3), (2, 3), (3, 4), (3, 4)]
    assert [tp.shard_kv_heads(p, s, 4, 2, r)[2:] for r in range(2)] == [(0, 2), (2, 4)]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K = 96, 512
        w = oc.synthetic_weight(M, K, seed=1)
        p, s = oc.encode(w)
        x = oc.synthetic_act(K, seed=2)
        full = oc.gemv_f64(p, s, x)
        # column parallel: rows split, all_gather of the outputs
        lo, hi = tp.split_range(M, world, rank, 16)
        ps, ss = tp.shard_rows(p, s, lo, hi)
        y_part = torch.from_numpy(oc.gemv_f64(ps, ss, x))
        outs = [torch.empty(r[1] - r[0], dtype=torch.float64)
                for r in (tp.split_range(M, world, i, 16) for i in range(world))]
        dist.all_gather(outs, y_part)
        col_ok = np.array_equal(torch.cat(outs).numpy(), full)
        # row parallel: K split, all_reduce of the partial sums
        pk, sk, k0, k1 = tp.shard_k(p, s, K, world, rank)
        part = torch.from_numpy(oc.gemv_f64(np.ascontiguousarray(pk), np.ascontiguousarray(sk),
                                            x[k0:k1]))
        dist.all_reduce(part)
        row_ok = np.allclose(part.numpy(), full, rtol=1e-12, atol=1e-12)
        # grouped rows ([q | k | v] with per-head units)
        groups = (32, 32, 32)
        pg, sg = tp.shard_grouped_rows(p, s, groups, 16, world, rank, np.concatenate)
        yg = oc.gemv_f64(pg, sg, x)
        want = np.concatenate([full[o + tp.split_range(n, world, rank, 16)[0]:
                                    o + tp.split_range(n, world, rank, 16)[1]]
                               for o, n in zip((0, 32, 64), groups)])
        grp_ok = np.array_equal(yg, want)
        q.put((rank, col_ok, row_ok, grp_ok))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharded_gemv_matches_full():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] and r[2] and r[3] for r in res), res

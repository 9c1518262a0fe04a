"""Tensor-parallel sharding of NVFP4 weights in the reference container's raw layout.

The reference is single-GPU; the partition follows the usual column/row split of a decoder:
projections that produce heads or MLP channels are split by OUTPUT ROWS (a contiguous byte range
of both arrays, because rows are contiguous), projections that consume them are split along K
(the same byte range of every row, repacked dense), and each K-split layer is followed by an
all-reduce of its 5120-element output.  Scale blocks (16 weights) and the kernels' K granularity
(128) never straddle ranks.

Layouts that concatenate several head groups are split per group:
  q_proj      rows are per head [q 256 | gate 256]      -> split by head (512-row units)
  in_proj_qkv rows are [q nk*128 | k nk*128 | v nv*128] -> each of the three parts split by head
All functions work on numpy arrays or torch tensors of bytes (they only index).
"""
from __future__ import annotations

K_GRAN = 128          # the tensor-core GEMV's K granularity


def split_range(n: int, world: int, rank: int, unit: int = 1):
    """[lo, hi) of rank's share of n items that come in indivisible groups of `unit`."""
    assert n % unit == 0
    groups = n // unit
    per, rem = divmod(groups, world)
    lo = rank * per + min(rank, rem)
    hi = lo + per + (1 if rank < rem else 0)
    return lo * unit, hi * unit


def shard_rows(packed, scales, lo: int, hi: int):
    """Rows [lo, hi) of a matrix: contiguous in both arrays."""
    return packed[lo:hi], scales[lo:hi]


def shard_k(packed, scales, K: int, world: int, rank: int):
    """K range of a row-parallel layer: columns [k0, k1) of every row, k0/k1 multiples of 128."""
    k0, k1 = split_range(K, world, rank, K_GRAN)
    return packed[:, k0 // 2:k1 // 2], scales[:, k0 // 16:k1 // 16], k0, k1


def shard_kv_heads(packed, scales, n_heads: int, world: int, rank: int, rows_per_head: int = 256):
    """K/V projections: heads are dealt to ranks; with more ranks than heads a head is REPLICATED
    on world / n_heads consecutive ranks (each of them needs it for its query heads)."""
    if world <= n_heads:
        lo, hi = split_range(n_heads, world, rank)
    else:
        assert world % n_heads == 0
        lo = rank // (world // n_heads)
        hi = lo + 1
    return shard_rows(packed, scales, lo * rows_per_head, hi * rows_per_head) + (lo, hi)


def shard_grouped_rows(packed, scales, group_sizes, unit: int, world: int, rank: int, cat):
    """A projection whose rows are several concatenated head groups (sizes in rows): take this
    rank's heads (`unit` rows each) from every group and concatenate them with `cat`."""
    ps, ss, off = [], [], 0
    for n in group_sizes:
        lo, hi = split_range(n, world, rank, unit)
        ps.append(packed[off + lo:off + hi])
        ss.append(scales[off + lo:off + hi])
        off += n
    return cat(ps), cat(ss)

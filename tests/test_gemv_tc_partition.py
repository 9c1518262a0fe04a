"""Host-side check of the tensor-core GEMV's work partition (csrc/gemv_tc.cu): the stages of all row
tiles, numbered tile-major, are cut into G equal contiguous ranges; per tile exactly one CTA
reduces (the one holding the tile's first stages, for which that segment is the last of its range),
every other CTA touching the tile stores into its own slot (tile + cta), and slot indices stay
below ntiles + G.  Pure integer arithmetic, restated from the kernel."""
import pytest


def partition(M, K, sms=148):
    ntiles, nk = (M + 127) // 128, K // 256
    total = ntiles * nk
    G = min(total, 2 * sms)
    return ntiles, nk, total, G


def cta_of(g, total, G):
    return ((g + 1) * G - 1) // total


@pytest.mark.parametrize("M,K", [
    (1, 256), (128, 256), (300, 512), (5120, 5120), (6144, 5120), (17408, 5120), (5120, 17408),
    (34816, 5120), (248320, 5120), (40000, 1024), (48, 5120), (8704, 5120), (5120, 8704), (129, 17408),
])
def test_every_tile_has_one_reducer_and_unique_slots(M, K):
    ntiles, nk, total, G = partition(M, K)
    assert total * (G + 1) < 2 ** 32
    starts = [b * total // G for b in range(G + 1)]
    assert all(starts[b + 1] > starts[b] for b in range(G))          # no empty range
    used = set()
    for b in range(G):
        g0, g1 = starts[b], starts[b + 1]
        for g in (g0, g1 - 1):
            assert cta_of(g, total, G) == b                          # the kernel's inverse map
        # segments of this CTA: maximal runs of stages of one tile
        segs = []
        g = g0
        while g < g1:
            tile = g // nk
            end = min((tile + 1) * nk, g1)
            segs.append((tile, g, end))
            g = end
        for i, (tile, a, e) in enumerate(segs):
            c_first, c_last = cta_of(tile * nk, total, G), cta_of((tile + 1) * nk - 1, total, G)
            assert c_first <= b <= c_last
            if c_first == c_last:
                continue                                             # whole tile in one CTA: direct store
            if b == c_first:
                # the reducer waits for the others only in the LAST segment of its range, so no CTA
                # that is waited for ever waits itself before it has stored
                assert i == len(segs) - 1
            else:
                slot = tile + b
                assert slot < ntiles + G and slot not in used
                used.add(slot)

"""Host logic of the tensor-core GEMM's schedule (no GPU): the ranges of k-blocks that a split last
wave deals out must cover every (tile, k-block) of the left-over tiles exactly once, every CTA may
start at most one segment inside a tile (its first), and the CTAs whose partial accumulators a tile's
owner adds are exactly those that hold the tile's remaining k-blocks.  The walk below restates the
device-side walk (SegmentWalk / the epilogue's peer count in csrc/gemm_tcgen05.cu) in Python."""
import pytest

from frame_public_b200 import capi

SMS = 148


def _segments(sched, cta):
    """Segments (tile, kb0, kb1) of the CTA that started `cta`-th: whole tiles first, then its range
    of the split part."""
    kbs, segs = sched["k_blocks"], []
    grid = SMS if sched["sk_units"] else min(SMS, max(sched["dp_tiles"], 1))
    t = cta
    while t < sched["dp_tiles"]:
        segs.append((t, 0, kbs))
        t += grid
    if sched["sk_units"] and cta < sched["sk_ctas"]:
        rng = sched["sk_ctas"] - 1 - cta     # ranges are handed out against the start order
        u = sched["sk_units"] * rng // sched["sk_ctas"]
        u1 = sched["sk_units"] * (rng + 1) // sched["sk_ctas"]
        while u < u1:
            tile = u // kbs
            kb0 = u - tile * kbs
            n = min(u1 - u, kbs - kb0)
            segs.append((sched["dp_tiles"] + tile, kb0, kb0 + n))
            u += n
    return segs


SHAPES = [(512, 1024, 8192, capi.BF16), (640, 1280, 8192, capi.BF16), (500, 520, 4104, capi.F32),
          (256, 512, 8192, capi.BF16), (1024, 1024, 2048, capi.F32), (128, 256, 65536, capi.BF16),
          (768, 1024, 32768, capi.F32)]


@pytest.mark.parametrize("m,n,k,dt", SHAPES, ids=lambda v: str(v))
def test_split_ranges_cover_every_k_block_once(m, n, k, dt):
    sched = capi.matmul_schedule(m, n, k, dt, compensated=(m, n, k) == (1024, 1024, 2048))
    assert sched["sk_units"] > 0, sched
    tiles = -(-m // sched["tile_m"]) * -(-n // sched["tile_n"])
    assert sched["dp_tiles"] % SMS == 0 and sched["dp_tiles"] < tiles
    assert sched["sk_units"] == (tiles - sched["dp_tiles"]) * sched["k_blocks"]
    assert 2 <= sched["sk_ctas"] <= SMS
    seen = {}
    for cta in range(SMS):
        segs = _segments(sched, cta)
        inside = [i for i, (_, kb0, _) in enumerate(segs) if kb0 > 0]
        first_split = next((i for i, s in enumerate(segs) if s[0] >= sched["dp_tiles"]), None)
        assert inside in ([], [first_split]), (cta, segs)   # one partial tile per CTA at most
        for tile, kb0, kb1 in segs:
            assert 0 <= kb0 < kb1 <= sched["k_blocks"]
            for kb in range(kb0, kb1):
                assert (tile, kb) not in seen, (tile, kb, cta, seen[(tile, kb)])
                seen[(tile, kb)] = cta
    assert len(seen) == tiles * sched["k_blocks"]
    # the owner of a tile (holder of k-block 0) finds the rest with the CTAs that started just BEFORE
    # it, in order: a CTA never waits for one that may not be running yet
    for tile in range(sched["dp_tiles"], tiles):
        owner = seen[(tile, 0)]
        holders = []
        for kb in range(sched["k_blocks"]):
            if not holders or holders[-1] != seen[(tile, kb)]:
                holders.append(seen[(tile, kb)])
        assert holders == list(range(owner, owner - len(holders), -1)), (tile, holders)


def test_full_machines_and_short_k_are_not_split():
    assert capi.matmul_schedule(8192, 8192, 8192, capi.BF16)["sk_units"] == 0      # 13.8 waves
    assert capi.matmul_schedule(32768, 1536, 48, capi.F32)["sk_units"] == 0        # two k-blocks
    assert capi.matmul_schedule(4096, 1024, 4096, capi.BF16)["sk_units"] == 0      # 128 tiles: L2-bound
    assert capi.matmul_schedule(2048, 8192, 8192, capi.BF16)["sk_units"] == 0      # 3.46 waves: measured no gain
    assert capi.matmul_schedule(64, 256, 784, capi.F32)["sk_units"] == 0           # 25 k-blocks
    s = capi.matmul_schedule(8192, 8192, 8192, capi.BF16, light_epilogue=True)
    assert (s["tile_m"], s["tile_n"], s["sk_units"]) == (256, 256, 0)
    # one wave of wide tiles rather than two of narrow ones
    assert capi.matmul_schedule(4096, 1024, 4096, capi.BF16)["tile_n"] == 256
    assert capi.matmul_schedule(4096, 1024, 1024, capi.BF16)["tile_n"] == 256
    assert capi.matmul_schedule(64, 512, 784, capi.F32)["tile_n"] == 128

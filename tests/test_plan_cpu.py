"""Host logic of the tensor-core path's work plans (no GPU: the library assumes 148 SMs without a device).

Which kernel takes which problem, when K is split, when the tiles are cut in balanced ranges, and - for
the balanced plan - that the ranges partition the (tile, k step) sequence exactly, that every cut tile has
one part that finishes it (its head, the LAST item of a unit) and that all its other parts belong to the
units that follow (each their FIRST item), which is what makes the in-kernel waits deadlock-free."""
import pytest

from gemmlib_b200 import capi

BIG = 1 << 30


def test_which_kernel_takes_which_problem():
    assert capi.gemm_plan(1, 11008, 4096)["kernel"] == "skinny"
    assert capi.gemm_plan(16, 4096, 4096)["kernel"] == "skinny"
    p = capi.gemm_plan(64, 28672, 8192, BIG)                 # 224 tiles on 148 SMs: balanced ranges
    assert (p["kernel"], p["rows_per_tile"], p["tiles"], p["balanced"], p["units"]) == ("one-cta", 64, 224, True, 148)
    assert not capi.gemm_plan(64, 28672, 8192, 0)["balanced"]  # no workspace: whole rounds
    p = capi.gemm_plan(2048, 4096, 4096, BIG)                # c3: 128 pair tiles on 74 pairs, 86 % busy
    assert (p["kernel"], p["rows_per_tile"], p["tiles"], p["balanced"], p["split"]) == ("pair", 256, 128, False, 1)
    p = capi.gemm_plan(512, 11008, 4096, BIG)                # 86 pair tiles: balanced
    assert (p["kernel"], p["tiles"], p["balanced"], p["units"]) == ("pair", 86, True, 74)
    p = capi.gemm_plan(512, 4096, 4096, BIG)                 # 32 pair tiles < 74 pairs: one-CTA kernel, split K
    assert (p["kernel"], p["tiles"], p["split"]) == ("one-cta", 64, 2)
    assert capi.gemm_plan(512, 4096, 4096, 0)["split"] == 1
    p = capi.gemm_plan(256, 4096, 4096, BIG)
    assert (p["kernel"], p["split"]) == ("one-cta", 4)
    assert capi.gemm_workspace_size(256, 4096, 4096) > capi.static_scratch_size()  # the shape the static entry refuses


@pytest.mark.parametrize("tiles,k_steps,units", [(224, 128, 148), (172, 64, 148), (86, 64, 74), (112, 128, 74),
                                                 (160, 16, 74), (448, 128, 74), (151, 8, 148), (300, 172, 148),
                                                 (32, 64, 74), (40, 172, 74)])
def test_balanced_ranges_partition_the_steps(tiles, k_steps, units):
    total = tiles * k_steps
    bounds = [capi.gemm_plan_range_bound(total, k_steps, units, b) for b in range(units + 1)]
    assert bounds[0] == 0 and bounds[-1] == total
    assert all(a <= b for a, b in zip(bounds, bounds[1:]))
    covered = [0] * total
    heads, others = {}, {}
    for u in range(units):
        pos, end, first = bounds[u], bounds[u + 1], True
        while pos < end:
            tile, ks0 = divmod(pos, k_steps)
            count = min(k_steps - ks0, end - pos)
            for s in range(pos, pos + count):
                covered[s] += 1
            if ks0 == 0 and count < k_steps:
                assert pos + count == end, "the head of a cut tile is the last item of its unit"
                heads[tile] = u
            elif ks0 > 0:
                assert first, "every other part of a cut tile is the first item of its unit"
                others.setdefault(tile, []).append(u)
            assert count >= min(4, k_steps) or count == end - pos or ks0 + count == k_steps
            pos += count
            first = False
    assert all(c == 1 for c in covered)
    assert set(heads) == set(others)
    for tile, u in heads.items():
        # the parts of a cut tile sit in consecutive units after the one that finishes it
        assert others[tile] == list(range(u + 1, u + 1 + len(others[tile])))


def test_which_shapes_the_fused_all_gather_takes():
    """blkq4_gather_supported_sm100 (per-rank shard shapes): decode and skinny shapes on the fast skinny
    paths, prefill shapes with at least one round of pair tiles, nothing in between."""
    assert capi.gather_supported(64, True, 1, 5504, 4096)        # decode kernel
    assert capi.gather_supported(128, True, 16, 3584, 8192)      # TMA skinny kernel
    assert not capi.gather_supported(32, True, 1, 4096, 4096)    # block 32: generic kernel
    assert not capi.gather_supported(64, False, 4, 4096, 4096)   # row-wise blocks
    assert not capi.gather_supported(64, True, 64, 14336, 8192)  # between the skinny and the pair kernel
    assert capi.gather_supported(128, True, 4096, 3584, 8192)    # 16 x 14 pair tiles >= 74 pairs
    assert not capi.gather_supported(128, True, 256, 3584, 8192)  # 14 pair tiles: not a round
    assert not capi.gather_supported(64, True, 512, 4100, 4096)  # N not a multiple of 16

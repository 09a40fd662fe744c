"""Planning of the two-pass backward's calls under a workspace bound (no GPU): every (batch, kv group) is covered once, no
range exceeds the bound unless it is a single group, and a range is either whole batches or groups of one batch."""
import itertools

import pytest

from delta_matching_b200.ops import plan_workspace_ranges

TILE = 16384 + 16


@pytest.mark.parametrize("B,Hk,rep,n_t", [(4, 8, 4, 32), (3, 2, 2, 8), (1, 1, 8, 256), (8, 8, 8, 16)])
@pytest.mark.parametrize("cap_groups", [0.5, 1, 1.5, 3, 8, 20, 1000])
def test_ranges_cover_all_units_within_the_bound(B, Hk, rep, n_t, cap_groups):
    group_bytes = rep * n_t * n_t * TILE
    cap = int(cap_groups * group_bytes)
    ranges = plan_workspace_ranges(B, Hk, rep, n_t, group_bytes, cap)
    seen = set()
    for b0, b1, g0, g1 in ranges:
        assert 0 <= b0 < b1 <= B and 0 <= g0 < g1 <= Hk
        assert (g0, g1) == (0, Hk) or b1 - b0 == 1                     # whole batches, or groups of one batch
        units = (b1 - b0) * (g1 - g0)
        assert units * group_bytes <= cap or units == 1
        assert units * rep * n_t * n_t < (1 << 24)
        for u in itertools.product(range(b0, b1), range(g0, g1)):
            assert u not in seen
            seen.add(u)
    assert len(seen) == B * Hk


def test_tile_limit_splits_long_contexts():
    # N = 131072 (n_t = 1024): one query head has 2^20 tiles, so at most 15 heads fit one call whatever the byte bound
    ranges = plan_workspace_ranges(1, 8, 4, 1024, 4 * 1024 * 1024 * TILE, 1 << 62)
    assert all((g1 - g0) * 4 * 1024 * 1024 < (1 << 24) for _, _, g0, g1 in ranges)
    assert sum(g1 - g0 for _, _, g0, g1 in ranges) == 8


def test_ranges_are_balanced():
    # 64 units with room for 9 per call: eight calls of eight, not seven of nine and one of one
    group_bytes = 8 * 256 * 256 * TILE
    ranges = plan_workspace_ranges(64, 1, 8, 256, group_bytes, 9 * group_bytes + 5)
    assert [b1 - b0 for b0, b1, _, _ in ranges] == [8] * 8
    ranges = plan_workspace_ranges(1, 8, 4, 32, 4 * 32 * 32 * TILE, 3 * 4 * 32 * 32 * TILE)
    assert sorted(g1 - g0 for _, _, g0, g1 in ranges) == [2, 3, 3]

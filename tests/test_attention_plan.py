"""How the tcgen05 prefill kernel's work is dealt to blocks: every query tile's key tiles are
walked exactly once, whether one block takes them all or several share them."""

import itertools

import pytest

from semantic_aware_adaptive_kv_cache_precision_b200.ops.attention import plan_wide_tiles

CASES = [
    ([0], [2048], 12, None),
    ([0, 37, 600, 299], [150, 91, 300, 1], 4, None),
    ([0, 100], [1100, 130], 7, 200),
    ([5000], [3000], 2, 700),
    ([0], [20000], 28, None),
]


@pytest.mark.parametrize("starts,counts,heads,window", CASES)
@pytest.mark.parametrize("slots", [1, 296, 10 ** 6])
def test_every_key_tile_once(starts, counts, heads, window, slots):
    work, folds, partials = plan_wide_tiles(starts, counts, heads, window, slots=slots)
    # the tiles as the kernel must see them
    want, row = {}, 0
    for i, (s, c) in enumerate(zip(starts, counts)):
        for a in range(0, c, 128):
            rows, pos0 = min(128, c - a), s + a
            first = max(0, pos0 - window + 1) // 64 if window else 0
            want[(i, row + a, rows, pos0)] = set(range(first, (pos0 + rows - 1) // 64 + 1))
        row += c
    seen = {k: [] for k in want}
    used = set()
    for (i, r0, rows, pos0, t0, n, partial, _) in work:
        assert n > 0
        seen[(i, r0, rows, pos0)].extend(range(t0, t0 + n))
        if partial >= 0:
            assert partial not in used and partial < partials
            used.add(partial)
    for key, tiles in seen.items():
        assert sorted(tiles) == sorted(want[key]) and len(set(tiles)) == len(tiles)
    assert used == set(range(partials))
    # each fold owns a run of partials that belong to one tile
    owned = list(itertools.chain.from_iterable(range(f[0], f[0] + f[1]) for f in folds))
    assert sorted(owned) == list(range(partials))
    by_partial = {w[6]: w for w in work if w[6] >= 0}
    for (first, count, r0, rows) in folds:
        assert count >= 2
        assert all(by_partial[p][1] == r0 and by_partial[p][2] == rows
                   for p in range(first, first + count))
    if slots == 1:
        assert not folds
    # the longest blocks come first
    assert [w[5] for w in work] == sorted((w[5] for w in work), reverse=True)


def test_many_blocks_are_left_whole():
    """A step with more blocks than run at once is not cut: the fold would cost more than
    the balance gains."""
    work, folds, partials = plan_wide_tiles([0], [4096], 12, None, slots=296)
    assert not folds and partials == 0
    work, folds, partials = plan_wide_tiles([0], [2048], 12, None, slots=296)
    assert folds and max(w[5] for w in work) <= 16

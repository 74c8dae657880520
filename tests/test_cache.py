"""Slots and blocks: nothing lost, nothing held twice, nothing freed twice. No GPU
(the cache's tensors are made on the CPU here; the bookkeeping is the same)."""

import numpy as np
import pytest
import torch

from semantic_aware_adaptive_kv_cache_precision_b200.cache import (BLOCK, CacheFull, KVNeed, Pool,
                                                                    SequenceCache, StateNeed)


def test_pool_take_and_give_back():
    pool = Pool(4, "slot")
    a = pool.take(3)
    assert a == [0, 1, 2] and pool.free == 1
    with pytest.raises(CacheFull, match="nothing was taken"):
        pool.take(2)
    assert pool.free == 1
    pool.give_back([1])
    assert pool.take(2) == [1, 3]
    with pytest.raises(RuntimeError, match="not held"):
        pool.give_back([1, 1])
    pool.give_back([0, 1, 2, 3])
    with pytest.raises(RuntimeError, match="not held"):
        pool.give_back([2])
    pool.check()
    assert pool.free == 4 and pool.held == 0


def make(max_tokens=640, window=None, state=False, max_positions=512):
    needs = [KVNeed(2, 16), KVNeed(2, 16), KVNeed(1, 32, window)]
    if state:
        needs.append(StateNeed((3, 4), "float32"))
    return SequenceCache(needs, max_tokens, max_positions, torch.float32, "cpu")


def test_groups_by_need():
    cache = make(window=100, state=True)
    assert len(cache.groups) == 2
    assert cache.groups[0].keys.shape == (2, 10, 2, BLOCK, 16)
    assert cache.groups[1].keys.shape == (1, 10, 1, BLOCK, 32)
    assert cache.states[3].shape == (cache.max_slots, 3, 4)
    view = cache.entry_view(1, ["t0", "t1"])
    assert view.keys.shape == (10, 2, BLOCK, 16) and view.block_table == "t0"
    assert cache.entry_view(2, ["t0", "t1"]).block_table == "t1"
    assert cache.entry_view(3, []).state is cache.states[3]


def test_reserve_is_all_or_nothing_and_lengths_are_per_sequence():
    cache = make(max_tokens=5 * BLOCK)
    a, b = cache.open(2)
    cache.reserve([a, b], [65, 100])
    assert cache.groups[0].pool.held == 4
    cache.advance([a, b], [65, 100])
    assert cache.lengths[a] == 65 and cache.lengths[b] == 100
    with pytest.raises(CacheFull):
        cache.reserve([a, b], [129, 129])         # needs 2 more, only 1 free
    assert cache.groups[0].pool.held == 4          # nothing was taken
    cache.reserve([a], [128])                      # still inside its second block
    assert cache.groups[0].pool.held == 4
    cache.reserve([a], [129])
    assert cache.groups[0].pool.held == 5
    cache.check()
    with pytest.raises(CacheFull, match="exceeds"):
        cache.reserve([a], [10 ** 6])


def test_slots_and_blocks_are_used_again():
    cache = make(max_tokens=4 * BLOCK)
    seen_blocks = set()
    for round_ in range(5):
        slots = cache.open(2)
        assert slots == [0, 1]
        cache.reserve(slots, [70, 30])
        cache.advance(slots, [70, 30])
        tables = cache.tables_for(slots)[0]
        used = tables[tables >= 0].tolist()
        assert len(used) == 3 and len(set(used)) == 3
        seen_blocks.update(used)
        cache.check()
        cache.close([slots[1]])                    # the shorter one ends first
        cache.check()
        assert cache.groups[0].pool.held == 2
        cache.close([slots[0]])
        assert cache.groups[0].pool.held == 0 and cache.slots.held == 0
    assert seen_blocks <= set(range(4))
    with pytest.raises(RuntimeError, match="not held"):
        cache.close([0])


def test_closing_twice_and_foreign_slots_fail():
    cache = make()
    (a,) = cache.open(1)
    cache.close([a])
    with pytest.raises(RuntimeError):
        cache.close([a])
    with pytest.raises(CacheFull):
        cache.open(cache.max_slots + 1)
    assert cache.slots.held == 0
    cache.check()


def test_window_group_gives_old_blocks_back():
    cache = make(max_tokens=10 * BLOCK, window=70)
    (a,) = cache.open(1)
    cache.reserve([a], [200])
    cache.advance([a], [200])
    full, windowed = cache.groups
    assert full.pool.held == 4
    # next query is at position 200 and sees keys 131..200: block 2 (128-191) on
    assert windowed.tables[a, :4].tolist()[:2] == [-1, -1] and windowed.pool.held == 2
    for n in range(201, 330):
        cache.reserve([a], [n])
        cache.advance([a], [n])
        cache.check()
        first_needed = max(0, n - 70 + 1) // BLOCK
        held = np.flatnonzero(windowed.tables[a] >= 0)
        assert held.min() == first_needed and held.max() == (n - 1) // BLOCK
    assert windowed.pool.held <= 3
    cache.close([a])
    assert windowed.pool.held == 0 and full.pool.held == 0
    cache.check()


def test_state_is_zeroed_when_a_slot_is_taken():
    cache = make(state=True)
    (a,) = cache.open(1)
    cache.states[3][a] = 7.0
    cache.close([a])
    (b,) = cache.open(1)
    assert a == b and float(cache.states[3][b].abs().sum()) == 0.0


def test_poisoned_blocks():
    cache = SequenceCache([KVNeed(1, 16)], 2 * BLOCK, 128, torch.float32, "cpu", poison_freed=True)
    (a,) = cache.open(1)
    cache.reserve([a], [10])
    block = int(cache.groups[0].tables[a, 0])
    cache.close([a])
    assert torch.isnan(cache.groups[0].keys[0, block]).all()
    assert not torch.isnan(cache.groups[0].keys[0, 1 - block]).any()


def test_keys_and_values_of_their_own_widths_and_type():
    """A need may give values another width than keys, no values at all, or a type of its
    own; entries with different needs get storage of their own."""
    needs = [KVNeed(2, 16), KVNeed(2, 16, value_dim=40), KVNeed(1, 24, value_dim=0),
             KVNeed(2, 16, dtype="float32"), KVNeed(2, 16, value_dim=40)]
    cache = SequenceCache(needs, 4 * BLOCK, 256, torch.bfloat16, "cpu", poison_freed=True)
    assert len(cache.groups) == 4
    by_need = {g.need: g for g in cache.groups}
    wide = by_need[KVNeed(2, 16, value_dim=40)]
    assert wide.keys.shape == (2, 4, 2, BLOCK, 16) and wide.values.shape == (2, 4, 2, BLOCK, 40)
    latent = by_need[KVNeed(1, 24, value_dim=0)]
    assert latent.values is None and latent.keys.shape == (1, 4, 1, BLOCK, 24)
    assert by_need[KVNeed(2, 16, dtype="float32")].keys.dtype == torch.float32
    assert by_need[KVNeed(2, 16)].keys.dtype == torch.bfloat16
    expected = sum(t.numel() * t.element_size() for g in cache.groups
                   for t in (g.keys, g.values) if t is not None)
    assert cache.nbytes == expected
    (a,) = cache.open(1)
    cache.reserve([a], [70])
    view = cache.entry_view(2, [torch.zeros(1, 2, dtype=torch.int32)] * 4)
    assert view.values is None and view.keys.shape == (4, 1, BLOCK, 24)
    view = cache.entry_view(4, [torch.zeros(1, 2, dtype=torch.int32)] * 4)
    assert view.values.shape == (4, 2, BLOCK, 40)
    cache.close([a])          # freed blocks are poisoned, the missing values are no obstacle
    cache.check()
    with pytest.raises(TypeError, match="dtype"):
        SequenceCache([KVNeed(1, 16, dtype="float16")], BLOCK, 64, torch.float32, "cpu")


def test_a_cache_the_device_cannot_hold_is_a_typed_error(monkeypatch):
    from semantic_aware_adaptive_kv_cache_precision_b200 import OutOfDeviceMemory
    real, calls = torch.zeros, []

    def no_room(*args, **kwargs):
        calls.append(args)
        if len(calls) == 3:           # the second group's keys: the first group is built
            raise torch.OutOfMemoryError("injected")
        return real(*args, **kwargs)

    monkeypatch.setattr(torch, "zeros", no_room)
    with pytest.raises(OutOfDeviceMemory, match="a cache of 4 blocks"):
        SequenceCache([KVNeed(2, 16), KVNeed(1, 32)], 4 * BLOCK, 256, torch.float32, "cpu")

"""The cache of live sequences.

Every live sequence holds a slot. Cache entries (one per layer call that writes
a cache) are sorted into groups by what they need:

* entries with the same `KVNeed` (heads, key and value widths, window, type) form a KV
  group with storage of its own: `keys` [entries, blocks, kv_heads, 64, head_dim] and
  `values` [..., value_dim], a pool of blocks, and for every slot the list of blocks that hold
  its positions 0-63, 64-127, ... A group with a window gives a sequence's
  blocks back as soon as every position in them has fallen out of the window.
* every entry with a `StateNeed` has a tensor [slots, *shape]: state of fixed
  size per sequence, zeroed when a slot is taken.

Each sequence has its own length. Storage is sized by `max_tokens`, the most
positions that live sequences hold at any time with each sequence's count
rounded up to a multiple of 64. The reference's caches hold one sequence
(`src/microinfer/model.py:95-132, 147-286`); slots, groups and state are this
library's own.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..errors import allocate
from .allocator import CacheFull, Pool
from .needs import KVNeed, StateNeed

BLOCK = 64

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class EntryView:
    """What one layer call sees of the cache during a step."""
    need: object
    keys: torch.Tensor | None = None          # [blocks, kv_heads, 64, head_dim]
    values: torch.Tensor | None = None        # [blocks, kv_heads, 64, value_dim]; None if 0
    block_table: torch.Tensor | None = None   # int32 [B, max_blocks], this step's sequences
    state: torch.Tensor | None = None         # [slots, *shape]; index with the step's slots
    group: int = -1


class KVGroup:
    def __init__(self, need: KVNeed, entries: list[int], blocks: int, max_blocks_per_seq: int,
                 max_slots: int, dtype: torch.dtype, device):
        self.need, self.entries = need, entries
        self.pool = Pool(blocks, "cache block")
        if need.dtype is not None:
            if need.dtype not in _DTYPES:
                raise TypeError(f"{need!r}: dtype must be one of {sorted(_DTYPES)} or None")
            dtype = _DTYPES[need.dtype]
        lead = (len(entries), max(blocks, 1), need.kv_heads, BLOCK)
        def zeros(width):
            shape = lead + (width,)
            count = int(np.prod(shape))
            return allocate(lambda: torch.zeros(shape, dtype=dtype, device=device),
                            f"a cache of {blocks} blocks of {BLOCK} positions for "
                            f"{len(entries)} layer(s)", count * dtype.itemsize)

        self.keys = zeros(need.head_dim)
        self.values = None if need.value_width == 0 else zeros(need.value_width)
        self.max_blocks_per_seq = max_blocks_per_seq
        # host copy of every slot's block list; -1 = no block
        self.tables = np.full((max_slots, max_blocks_per_seq), -1, dtype=np.int32)


class SequenceCache:
    """Slots, blocks, lengths and per-sequence state of all live sequences."""

    def __init__(self, needs: list, max_tokens: int, max_positions: int, dtype: torch.dtype,
                 device, max_slots: int | None = None, poison_freed: bool = False):
        if max_tokens <= 0:
            raise ValueError(f"max_tokens must be positive, got {max_tokens}")
        self.dtype, self.device = dtype, torch.device(device)
        self.blocks = -(-max_tokens // BLOCK)
        self.max_tokens = self.blocks * BLOCK
        self.max_seq_len = min(max_positions, self.max_tokens)
        self.max_blocks_per_seq = -(-self.max_seq_len // BLOCK)
        self.max_slots = max_slots if max_slots is not None else min(self.blocks, 1024)
        self.poison_freed = poison_freed
        self.slots = Pool(self.max_slots, "sequence slot")
        self.lengths = np.zeros(self.max_slots, dtype=np.int64)
        self.needs = list(needs)
        self.groups: list[KVGroup] = []
        self.entry_group: dict[int, tuple[int, int]] = {}     # entry -> (group, index in group)
        self.states: dict[int, torch.Tensor] = {}
        by_need: dict[KVNeed, list[int]] = {}
        for entry, need in enumerate(self.needs):
            if isinstance(need, KVNeed):
                by_need.setdefault(need, []).append(entry)
            elif isinstance(need, StateNeed):
                shape = (self.max_slots,) + tuple(need.shape)
                self.states[entry] = allocate(
                    lambda: torch.zeros(shape, dtype=_DTYPES[need.dtype], device=device),
                    f"the per-sequence state of cache entry {entry}",
                    int(np.prod(shape)) * _DTYPES[need.dtype].itemsize)
            elif need is not None:
                raise TypeError(f"cache entry {entry}: unknown need {need!r}")
        for need, entries in by_need.items():
            g = len(self.groups)
            self.groups.append(KVGroup(need, entries, self.blocks, self.max_blocks_per_seq,
                                       self.max_slots, dtype, device))
            for i, entry in enumerate(entries):
                self.entry_group[entry] = (g, i)
        # first position whose block a window group still holds, per (group, slot)
        self._front = [np.zeros(self.max_slots, dtype=np.int64) for _ in self.groups]

    # -- sizes --------------------------------------------------------------

    @property
    def nbytes(self) -> int:
        total = sum(t.numel() * t.element_size() for g in self.groups
                    for t in (g.keys, g.values) if t is not None)
        return total + sum(s.numel() * s.element_size() for s in self.states.values())

    # -- slots --------------------------------------------------------------

    def open(self, count: int = 1) -> list[int]:
        """Take `count` slots (all or none) for sequences of length 0."""
        slots = self.slots.take(count)
        for s in slots:
            self.lengths[s] = 0
            for g, group in enumerate(self.groups):
                group.tables[s, :] = -1
                self._front[g][s] = 0
        if slots and self.states:
            index = torch.as_tensor(slots, dtype=torch.long, device=self.device)
            for state in self.states.values():
                state.index_fill_(0, index, 0)
        return slots

    def close(self, slots) -> None:
        """End sequences: their blocks and slots go back to the pools."""
        slots = list(slots)
        for s in slots:
            if s not in self.slots._held:
                raise RuntimeError(f"slot {s} is not held (closed twice, or never opened)")
        for s in slots:
            for g, group in enumerate(self.groups):
                row = group.tables[s]
                self._release(group, [int(b) for b in row[row >= 0]])
                row[:] = -1
            self.lengths[s] = 0
        self.slots.give_back(slots)

    def _release(self, group: KVGroup, blocks: list[int]) -> None:
        if not blocks:
            return
        if self.poison_freed and group.keys.is_floating_point():
            index = torch.as_tensor(blocks, dtype=torch.long, device=self.device)
            group.keys.index_fill_(1, index, float("nan"))
            if group.values is not None:
                group.values.index_fill_(1, index, float("nan"))
        group.pool.give_back(blocks)

    # -- growth -------------------------------------------------------------

    def reserve(self, slots, new_lengths) -> None:
        """Make room for every sequence `slots[i]` to reach `new_lengths[i]`
        positions. All or nothing: if any group lacks blocks, or a sequence would
        pass the longest length the cache takes, nothing changes."""
        plans = []
        for g, group in enumerate(self.groups):
            want = []
            for s, n in zip(slots, new_lengths):
                if n > self.max_seq_len:
                    raise CacheFull(f"a sequence of {n} positions exceeds the {self.max_seq_len} "
                                    "that this cache takes per sequence; nothing was taken")
                first = int(self._front[g][s]) // BLOCK
                last = -(-int(n) // BLOCK)
                missing = [b for b in range(first, last) if group.tables[s, b] < 0]
                want.append((s, missing))
            total = sum(len(m) for _, m in want)
            if total > group.pool.free:
                raise CacheFull(f"{total} cache block(s) of {BLOCK} positions needed, "
                                f"{group.pool.free} of {group.pool.size} free; nothing was taken")
            plans.append((group, want))
        for group, want in plans:
            for s, missing in want:
                for b, block in zip(missing, group.pool.take(len(missing))):
                    group.tables[s, b] = block

    def advance(self, slots, new_lengths) -> None:
        """Record the new lengths after a step; window groups give back the blocks
        whose positions no later query can see."""
        for s, n in zip(slots, new_lengths):
            self.lengths[s] = n
            for g, group in enumerate(self.groups):
                w = group.need.window
                if not w:
                    continue
                first_seen = max(0, int(n) - w + 1)       # oldest position the next query sees
                keep_from = first_seen // BLOCK
                old = int(self._front[g][s]) // BLOCK
                if keep_from > old:
                    row = group.tables[s]
                    gone = [int(b) for b in row[old:keep_from] if b >= 0]
                    row[old:keep_from] = -1
                    self._release(group, gone)
                    self._front[g][s] = keep_from * BLOCK

    # -- what a step sees -----------------------------------------------------

    def tables_for(self, slots) -> list[np.ndarray]:
        """For each KV group, the block lists of `slots` as int32 [B, max_blocks]."""
        index = np.asarray(list(slots), dtype=np.int64)
        return [group.tables[index] for group in self.groups]

    def entry_view(self, entry: int, device_tables: list) -> EntryView:
        need = self.needs[entry]
        if isinstance(need, KVNeed):
            g, i = self.entry_group[entry]
            group = self.groups[g]
            return EntryView(need, group.keys[i],
                             None if group.values is None else group.values[i],
                             device_tables[g], None, g)
        if isinstance(need, StateNeed):
            return EntryView(need, state=self.states[entry])
        return EntryView(need)

    def check(self) -> None:
        """Bookkeeping invariants: no slot or block lost, held twice or freed twice."""
        self.slots.check()
        for group in self.groups:
            group.pool.check()
            listed = group.tables[group.tables >= 0].tolist()
            if len(set(listed)) != len(listed):
                raise RuntimeError("a cache block is listed for two places")
            if set(listed) != group.pool._held:
                raise RuntimeError("held blocks and listed blocks differ: "
                                   f"{sorted(group.pool._held ^ set(listed))}")
            for s in range(self.max_slots):
                if s not in self.slots._held and (group.tables[s] >= 0).any():
                    raise RuntimeError(f"free slot {s} still lists blocks")

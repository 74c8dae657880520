"""Slots, blocks and per-sequence state of live sequences."""

from .allocator import CacheFull, Pool
from .needs import KVNeed, StateNeed
from .cache import BLOCK, EntryView, KVGroup, SequenceCache

__all__ = ["BLOCK", "CacheFull", "Pool", "KVNeed", "StateNeed", "EntryView", "KVGroup",
           "SequenceCache"]

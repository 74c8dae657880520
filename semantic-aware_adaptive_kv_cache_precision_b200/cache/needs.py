"""What a mixer asks of the cache, as data."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class KVNeed:
    """Keys and values that grow with the sequence: for each position `kv_heads x
    head_dim` of keys and `kv_heads x value_dim` of values. `window` None keeps every
    position; a number keeps the last `window` positions (older blocks are given back
    while the sequence runs).

    `value_dim` None: values as wide as keys (the usual attention). Another number: values
    of their own width (a mixer whose values are narrower or wider than its keys). 0: no
    values at all; the entry is one tensor per position (a mixer that caches a single
    latent and makes keys and values from it). `dtype` None: the type of the activations;
    'float32', 'bfloat16' or 'int32' fixes it whatever the engine's mode. Entries with the
    same need share a group, that is, a block pool and block lists."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None
    dtype: Optional[str] = None

    @property
    def value_width(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per sequence (a recurrent mixer's running state):
    a tensor of `shape` and `dtype` ('float32', 'bfloat16', 'int32') for each
    live sequence, zero when the sequence starts."""
    shape: tuple
    dtype: str = "float32"

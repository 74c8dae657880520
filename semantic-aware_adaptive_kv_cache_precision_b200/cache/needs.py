"""What a mixer asks of the cache, as data."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class KVNeed:
    """Keys and values that grow with the sequence: `kv_heads x head_dim` of each
    per position. `window` None keeps every position; a number keeps the last
    `window` positions (older blocks are given back while the sequence runs)."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per sequence (a recurrent mixer's running state):
    a tensor of `shape` and `dtype` ('float32', 'bfloat16', 'int32') for each
    live sequence, zero when the sequence starts."""
    shape: tuple
    dtype: str = "float32"

"""How a part says which tensors it needs from a checkpoint."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class TensorDecl:
    """One tensor a part reads, by its full name in the checkpoint.

    `init` says how the random-weights mode fills it: "normal" (N(0, std)),
    "ones_normal" (1 + N(0, std), for norm weights) or "zeros".
    `group`: tensors with the same group name, declared one after another,
    with equal trailing sizes and equal stored types, are laid back to back in
    device memory, so that the part can use them as one tensor (a fused
    q/k/v or gate/up matrix) without a copy.
    `integer`: a table of integers (kept as int32) rather than of numbers.
    """
    name: str
    shape: tuple
    init: str = "normal"
    group: Optional[str] = None
    integer: bool = False

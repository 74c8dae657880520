"""What every part of a model must offer, and the registry of part classes.

A part is built from a spec (`config.specs`) and the prefix of its tensors in
the checkpoint. It declares its tensors, picks them up from the weight arena
once they are loaded, and runs on the device. It is given everything it needs
as arguments; it never looks at a model or at a config.json.

Interfaces
----------
Norm            forward(x_fp32 [T, H], out_dtype, rows=None) -> [T or R, H]
PositionEncoding rotate_store(qkv, step, view, heads, kv_heads, head_dim, write_cache)
                rotates queries (in place) and keys, and stores keys and values in
                the cache entry `view`
Mixer           cache_need() -> KVNeed | StateNeed | None
                forward(h [T, H], step, view, residual_fp32 [T, H], write_cache)
                adds its output into `residual`
FeedForward     forward(h [T, H], step, residual_fp32 [T, H]); adds into `residual`
Block           forward(x_fp32 [T, H], step, view, write_cache); updates x in place

`step` is the `engine.step.StepContext` of the running step: the step's tokens,
positions, sequences and block tables on the device. `view` is the
`cache.EntryView` of the cache entry that this layer call reads or writes.

Steps whose shape repeats are captured in CUDA graphs and replayed. A replay
repeats the launches of the capture, Python numbers included; only what lies on
the device is fresh (`token_ids`, `positions`, `token_seq`, `seq_lens`, `slots`,
`want`, the block tables). Of the host-side facts, a graph is keyed by
`new_counts` and, for a model with per-sequence state, by `host_slots`; a
prefill graph also by `starts`. A part whose launches depend on anything else on
the host (`starts`, `max_position` or `max_len` in a decode step, or a value read
back from the device) sets `graph_safe = False`.
"""

from __future__ import annotations

import torch

from ..weights.decl import TensorDecl

_PARTS: dict[str, type] = {}


def register_part(kind: str, cls: type) -> None:
    """Make specs with `spec.kind == kind` build `cls(spec, prefix, mode)`."""
    _PARTS[kind] = cls


def build_part(spec, prefix: str, mode: str):
    kind = getattr(spec, "kind", None)
    if kind not in _PARTS:
        raise KeyError(f"no part is registered for kind {kind!r}; known kinds: "
                       f"{', '.join(sorted(_PARTS))}")
    return _PARTS[kind](spec, prefix, mode)


class Part:
    """Base of all parts. `mode` is 'bfloat16' or 'float32': the type of
    activations between kernels (the residual stream is fp32 in both)."""

    #: False for a part whose step cannot be captured in a CUDA graph (it synchronises with
    #: the host, or launches work whose shape depends on the data). The engine then runs
    #: decode steps kernel by kernel; it also falls back by itself if a capture fails.
    graph_safe = True

    def __init__(self, spec, prefix: str, mode: str):
        self.spec, self.prefix, self.mode = spec, prefix, mode
        self.act_dtype = torch.float32 if mode == "float32" else torch.bfloat16

    def tensor_decls(self) -> list[TensorDecl]:
        return []

    def bind(self, arena) -> None:
        """Pick up this part's tensors from the loaded arena."""

    def prepare(self, device, max_positions: int) -> None:
        """Build what depends on the device or on the longest sequence (tables)."""

"""One step's description on the device.

A step feeds some new tokens of each of B sequences through the model: whole
prompts of unequal length (prefill), or one token each (decode). Its tokens are
packed one sequence after the other, without padding. For every token the
device needs its id, its position in its sequence and which sequence of the
batch it belongs to; for every sequence its length after the step and, for each
cache group, its list of blocks. All of this is assembled on the host into one
int32 buffer in pinned memory and sent with a single copy; the fields are views
into the device copy. The reference uploads ids and positions of its one
sequence per step (`src/microinfer/model.py:351-352`).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import BLOCK     # positions per cache block: block lists are counted in it


@dataclass
class StepContext:
    tokens: int                       # T, tokens in this step
    sequences: int                    # B
    token_ids: torch.Tensor           # int32 [T]
    positions: torch.Tensor           # int32 [T]
    token_seq: torch.Tensor           # int32 [T]: index into this step's sequences
    cu_seqlens: torch.Tensor          # int32 [B + 1]: where each sequence's tokens start
    seq_lens: torch.Tensor            # int32 [B]: length of each sequence after the step
    slots: torch.Tensor               # int32 [B]: cache slot of each sequence
    want: torch.Tensor                # int32 [W]: token rows whose logits are wanted
    tables: list                      # per KV group: int32 [B, max_blocks]
    # host-side facts, for choosing kernels and checking bounds
    new_counts: list = field(default_factory=list)
    starts: list = field(default_factory=list)
    host_slots: list = field(default_factory=list)
    max_position: int = 0
    max_new: int = 0
    max_len: int = 0
    is_decode: bool = False           # every sequence brings exactly one token
    max_len_bound: int = 0            # a bound on max_len that changes rarely (block-list width)
    plans: dict = field(default_factory=dict)   # what a part worked out for this step, for its
                                                # other layers to use again (key chosen by the part)


class StepStager:
    """Pinned host buffers and the device buffer that carry a step's integers. There are two
    host buffers, used in turn: a step can be written while the copy of the step before it
    is still on its way (a decode loop that runs ahead of the tokens it has read back)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.capacity = 0
        self.hosts = [None, None]
        self.dev = None
        self.copied = [None, None]
        self.turn = 0
        self.last_bytes = 0
        self.generation = 0

    def _ensure(self, count: int) -> None:
        if count <= self.capacity:
            return
        self.capacity = max(1 << 18, 2 * count)
        self.generation += 1                 # device addresses change: captured graphs are stale
        self.hosts = [torch.empty(self.capacity, dtype=torch.int32, pin_memory=True)
                      for _ in range(2)]
        self.dev = torch.empty(self.capacity, dtype=torch.int32, device=self.device)
        self.copied = [None, None]

    def build(self, slots: list, new_tokens: list, starts: list, want_rows, tables: list,
              device_tokens: torch.Tensor | None = None) -> StepContext:
        """`new_tokens[i]`: the tokens sequence i brings; `starts[i]`: its length
        before the step; with `device_tokens` (int32 [B] on the device, one token a sequence)
        the ids are taken from there, on the stream, and `new_tokens` gives the counts only
        (if they ARE this stager's own token field, where a captured step's choice of tokens
        was written, they stay where they are and nothing is copied over them);
        `want_rows`: flat token rows whose logits are wanted;
        `tables[g]`: numpy int32 [B, max_blocks] of cache group g."""
        B = len(slots)
        counts = [len(t) for t in new_tokens]
        T = int(sum(counts))
        want_rows = np.asarray(want_rows, dtype=np.int32).reshape(-1)
        W = want_rows.size
        # block lists only as wide as the longest sequence of the step needs
        ends = [s + c for s, c in zip(starts, counts)]
        # (rounded up to a multiple of 8 blocks, so that a decode loop keeps one shape for
        # 512 steps and its captured graph can be replayed)
        width = -(-max(1, -(-max(ends, default=1) // BLOCK)) // 8) * 8
        tables = [np.ascontiguousarray(t[:, :min(width, t.shape[1])]) for t in tables]
        fields = [("token_ids", T), ("positions", T), ("token_seq", T), ("cu_seqlens", B + 1),
                  ("seq_lens", B), ("slots", B), ("want", W)]
        fields += [(f"table{g}", t.size) for g, t in enumerate(tables)]
        offsets, total = {}, 0
        for name, n in fields:
            offsets[name] = total
            total += -(-max(n, 1) // 4) * 4          # 16-byte aligned fields
        self._ensure(total)
        turn = self.turn = 1 - self.turn
        if self.copied[turn] is not None:
            self.copied[turn].synchronize()         # its last copy has left this host buffer
        host = self.hosts[turn].numpy()

        def put(name, values):
            values = np.asarray(values, dtype=np.int32).reshape(-1)
            host[offsets[name]:offsets[name] + values.size] = values

        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(counts, out=cu[1:])
        put("token_ids", np.zeros(T) if device_tokens is not None else
            np.concatenate([np.asarray(t, dtype=np.int64) for t in new_tokens]) if T
            else np.zeros(0))
        put("positions", np.concatenate([np.arange(s, s + c) for s, c in zip(starts, counts)])
            if T else np.zeros(0))
        put("token_seq", np.repeat(np.arange(B), counts))
        put("cu_seqlens", cu)
        put("seq_lens", [s + c for s, c in zip(starts, counts)])
        put("slots", slots)
        put("want", want_rows)
        for g, t in enumerate(tables):
            put(f"table{g}", t)
        in_place = (device_tokens is not None and offsets["token_ids"] == 0
                    and device_tokens.data_ptr() == self.dev.data_ptr())
        first = offsets["positions"] if in_place else 0      # (the token field comes first)
        self.last_bytes = 4 * (total - first)
        self.dev[first:total].copy_(self.hosts[turn][first:total], non_blocking=True)
        self.copied[turn] = torch.cuda.Event()
        self.copied[turn].record()
        if device_tokens is not None and not in_place:
            self.dev[offsets["token_ids"]:offsets["token_ids"] + T].copy_(device_tokens)

        def view(name, n):
            return self.dev[offsets[name]:offsets[name] + n]

        dev_tables = [view(f"table{g}", t.size).view(t.shape) for g, t in enumerate(tables)]
        return StepContext(
            tokens=T, sequences=B, token_ids=view("token_ids", T), positions=view("positions", T),
            token_seq=view("token_seq", T), cu_seqlens=view("cu_seqlens", B + 1),
            seq_lens=view("seq_lens", B), slots=view("slots", B), want=view("want", W),
            tables=dev_tables, new_counts=counts, starts=list(starts), host_slots=list(slots),
            max_position=max(ends) - 1 if ends else 0, max_new=max(counts, default=0),
            max_len=max(ends, default=0), is_decode=all(c == 1 for c in counts),
            max_len_bound=min(width, max((t.shape[1] for t in tables), default=width)) * BLOCK)

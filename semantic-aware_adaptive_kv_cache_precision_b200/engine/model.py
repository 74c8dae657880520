"""A decoder model built from a `ModelSpec`: embedding, blocks in their run
order, final norm, output head. It owns no sizes of its own: everything comes
from the spec, and every block is built from its part specs through the part
registry. The forward pass is the reference's `Model.run`
(`src/microinfer/model.py:345-403`) over a batch of sequences."""

from __future__ import annotations

import torch

from .. import ops
from ..parts import build_part
from ..weights import TensorDecl, load_checkpoint, random_arena


class DecoderModel:
    def __init__(self, spec, mode: str = "bfloat16", device="cuda"):
        if mode not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {mode!r}")
        self.spec, self.mode, self.device = spec, mode, torch.device(device)
        self.act_dtype = torch.float32 if mode == "float32" else torch.bfloat16
        self.blocks = [build_part(b, b.prefix, mode) for b in spec.blocks]
        self.final_norm = build_part(spec.final_norm, _strip(spec.final_norm_name), mode)
        owners = {}
        for call in spec.run_order:
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"run order names block {call.block}, the model has "
                                 f"{len(self.blocks)}")
            owners.setdefault(call.cache, call.block)
        if sorted(owners) != list(range(len(owners))):
            raise ValueError("cache entries of the run order must be numbered 0, 1, 2, ...")
        self._owners = owners
        self.arena = None
        #: whether every part says its step can be captured in a CUDA graph
        self.graph_safe = all(getattr(b, "graph_safe", True) for b in self.blocks)

    # -- tensors ----------------------------------------------------------------

    def tensor_decls(self) -> list[TensorDecl]:
        spec = self.spec
        decls = [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden))]
        for block in self.blocks:
            decls += block.tensor_decls()
        decls += self.final_norm.tensor_decls()
        if not spec.tie_head:
            decls.append(TensorDecl(spec.head_name, (spec.vocab_size, spec.hidden)))
        if spec.head_bias_name:
            decls.append(TensorDecl(spec.head_bias_name, (spec.vocab_size,), init="zeros"))
        return decls

    @staticmethod
    def tensor_decls_of(spec) -> list[TensorDecl]:
        """The declarations without a device (for writing random checkpoints)."""
        return DecoderModel(spec, "float32", "cpu").tensor_decls()

    def load(self, folder) -> None:
        self._bind(load_checkpoint(folder, self.tensor_decls(), self.mode, self.device,
                                   ignore=self.spec.ignore_tensors))

    def load_random(self, seed: int) -> None:
        self._bind(random_arena(self.tensor_decls(), seed, self.spec.init_std, self.mode,
                                self.device, self.spec.stored_dtype))

    def _bind(self, arena) -> None:
        self.embed = arena.view(self.spec.embed_name)
        self.head = self.embed if self.spec.tie_head else arena.view(self.spec.head_name)
        self.head_bias = arena.view(self.spec.head_bias_name) if self.spec.head_bias_name else None
        for block in self.blocks:
            block.bind(arena)
        self.final_norm.bind(arena)
        self.arena = arena

    @property
    def weight_bytes(self) -> int:
        return 0 if self.arena is None else self.arena.nbytes

    # -- cache ------------------------------------------------------------------

    def cache_needs(self) -> list:
        """What each cache entry must hold: the need of the block that owns it."""
        return [self.blocks[self._owners[e]].cache_need() for e in range(len(self._owners))]

    def prepare(self, max_positions: int) -> None:
        for block in self.blocks:
            block.prepare(self.device, max_positions)

    # -- the forward pass ---------------------------------------------------------

    def hidden(self, step, cache, capture: list | None = None) -> torch.Tensor:
        """The residual stream [T, hidden] (fp32) after the last layer call; the
        cache entries that the calls own are extended by the step's tokens.

        With `capture` (a list), copies of the stream are appended to it: after the
        embedding and after every layer call but the last, the order in which the
        reference captures hidden states (`src/microinfer/model.py:355-364, 398-402`);
        `final_states` gives the entry that closes that list."""
        if self.arena is None:
            raise RuntimeError("no weights on the device; load a checkpoint first")
        x = ops.embed(step.token_ids, self.embed)
        if self.spec.embed_scale != 1.0:
            ops.scale_cap_(x, self.spec.embed_scale)
        if capture is not None:
            capture.append(x.clone())
        written = set()
        pending = None          # a block's last output, not yet added to the stream
        last = len(self.spec.run_order) - 1
        for i, call in enumerate(self.spec.run_order):
            view = cache.entry_view(call.cache, step.tables)
            block = self.blocks[call.block]
            if getattr(block, "carries_pending", False):
                pending = block.forward(x, step, view, call.cache not in written, pending,
                                        leave_pending=i < last and capture is None)
            else:
                if pending is not None:
                    ops.add_into(x, pending)
                block.forward(x, step, view, call.cache not in written)
                pending = None
            written.add(call.cache)
            if capture is not None and i < last:
                capture.append(x.clone())
        if pending is not None:
            ops.add_into(x, pending)
        return x

    def final_states(self, x: torch.Tensor) -> torch.Tensor:
        """The stream after the final norm, fp32 [T, hidden]: the last entry of the captured
        hidden states."""
        return self.final_norm.forward(x, out_dtype=torch.float32)

    def logits(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """fp32 logits [len(rows), vocab] of the token rows `rows` of `x`: only
        these rows go through the final norm and the output head."""
        normed = self.final_norm.forward(x, rows=rows)
        out = ops.linear(normed, self.head, self.head_bias, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0 or self.spec.logit_softcap:
            ops.scale_cap_(out, self.spec.logit_scale, self.spec.logit_softcap)
        return out


def _strip(name: str) -> str:
    return name[:-len(".weight")] if name.endswith(".weight") else name

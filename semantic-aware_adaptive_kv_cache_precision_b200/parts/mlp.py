"""Dense gated feed-forward: `residual += down( silu(gate(h)) * up(h) )`
(`src/microinfer/model.py:392-396`, `src/core_kernels/swiglu.cu:26-38`). Gate and
up are one product over the rows [Wgate; Wup] laid back to back in device
memory; the activation is fp32 inside with one rounding at its store."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.decl import TensorDecl
from .base import Part, register_part


class GatedMLP(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r}: only 'silu' is built")
        if spec.bias:
            raise ValueError("a gated feed-forward with biases is not built")

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        return [TensorDecl(f"{p}gate_proj.weight", (s.intermediate, s.hidden), group=p + "gate_up"),
                TensorDecl(f"{p}up_proj.weight", (s.intermediate, s.hidden), group=p + "gate_up"),
                TensorDecl(f"{p}down_proj.weight", (s.hidden, s.intermediate))]

    def bind(self, arena):
        p = self.prefix
        self.w_gate_up = arena.group_view(p + "gate_up")
        if self.w_gate_up is None:
            self.w_gate_up = torch.cat([arena.view(p + "gate_proj.weight"),
                                        arena.view(p + "up_proj.weight")])
        self.w_down = arena.view(p + "down_proj.weight")

    can_defer = True

    def forward(self, h, step, residual, defer=False):
        act = ops.gated_up(h, self.w_gate_up)
        out = ops.linear(act, self.w_down, accumulate_into=residual, may_defer=defer)
        return out.delta if isinstance(out, ops.Deferred) else None


register_part("gated_mlp", GatedMLP)

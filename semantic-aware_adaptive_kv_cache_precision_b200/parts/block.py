"""The pre-norm arrangement of a layer: `x += mixer(norm(x)); x += ffn(norm(x))`
with the residual stream `x` in fp32 from the embedding to the final norm
(`src/microinfer/model.py:366-399`; `docs/adr/0010-the-residual-stream-is-fp32.md`)."""

from __future__ import annotations

from .. import ops
from .base import Part, build_part, register_part


class PreNormBlock(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        p = spec.prefix
        self.mixer_norm = build_part(spec.mixer_norm, p + spec.mixer_norm_name, mode)
        self.mixer = build_part(spec.mixer, p + spec.mixer_name + ".", mode)
        self.ffn_norm = build_part(spec.ffn_norm, p + spec.ffn_norm_name, mode)
        self.ffn = build_part(spec.ffn, p + spec.ffn_name + ".", mode)
        self.parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts)

    def tensor_decls(self):
        return [d for part in self.parts for d in part.tensor_decls()]

    def bind(self, arena):
        for part in self.parts:
            part.bind(arena)

    def prepare(self, device, max_positions):
        for part in self.parts:
            part.prepare(device, max_positions)

    def cache_need(self):
        return self.mixer.cache_need()

    # A mixer or feed-forward with `can_defer` may hand back its fp32 output instead of adding
    # it to the stream (`defer=True`); the norm that reads the stream next adds it on its way
    # if it has `folds_add`, so the stream is read and written once instead of twice. What the
    # feed-forward hands back leaves the block as `pending`: whoever runs the blocks gives it
    # to the next one, or asks the last one not to leave any (`leave_pending=False`).
    carries_pending = True

    def forward(self, x, step, view, write_cache=True, pending=None, leave_pending=True):
        h = _normed(self.mixer_norm, x, pending)
        if getattr(self.mixer, "can_defer", False):
            pending = self.mixer.forward(h, step, view, x, write_cache, defer=True)
        else:
            self.mixer.forward(h, step, view, x, write_cache)
            pending = None
        h = _normed(self.ffn_norm, x, pending)
        if leave_pending and getattr(self.ffn, "can_defer", False):
            return self.ffn.forward(h, step, x, defer=True)
        self.ffn.forward(h, step, x)
        return None


def _normed(norm, x, pending):
    if pending is None:
        return norm.forward(x)
    if getattr(norm, "folds_add", False):
        return norm.forward(x, add=pending)
    ops.add_into(x, pending)
    return norm.forward(x)


register_part("pre_norm", PreNormBlock)

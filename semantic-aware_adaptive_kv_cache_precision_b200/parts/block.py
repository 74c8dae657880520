"""The pre-norm arrangement of a layer: `x += mixer(norm(x)); x += ffn(norm(x))`
with the residual stream `x` in fp32 from the embedding to the final norm
(`src/microinfer/model.py:366-399`; `docs/adr/0010-the-residual-stream-is-fp32.md`)."""

from __future__ import annotations

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

    def forward(self, x, step, view, write_cache=True):
        self.mixer.forward(self.mixer_norm.forward(x), step, view, x, write_cache)
        self.ffn.forward(self.ffn_norm.forward(x), step, x)


register_part("pre_norm", PreNormBlock)

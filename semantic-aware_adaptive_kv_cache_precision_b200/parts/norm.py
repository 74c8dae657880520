"""RMSNorm: `x * rsqrt(mean(x^2) + eps) * w` over rows of the fp32 residual
stream (`src/core_kernels/rmsnorm.cu:33-84`; the weight multiplies directly)."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.decl import TensorDecl
from .base import Part, register_part


class RMSNorm(Part):
    """`prefix` is the tensor's name without '.weight'."""

    def tensor_decls(self):
        return [TensorDecl(self.prefix + ".weight", (self.spec.size,), init="ones_normal")]

    def bind(self, arena):
        self.weight = arena.view(self.prefix + ".weight")

    folds_add = True     # forward(x, add=delta) does x += delta on its way

    def forward(self, x, out_dtype=None, rows=None, add=None):
        out_dtype = out_dtype or self.act_dtype
        if add is not None and (rows is not None or out_dtype != torch.bfloat16
                                or self.weight.dtype != torch.bfloat16):
            ops.add_into(x, add)
            add = None
        return ops.rms_norm(x, self.weight, self.spec.eps, out_dtype, rows, add)


register_part("rms_norm", RMSNorm)

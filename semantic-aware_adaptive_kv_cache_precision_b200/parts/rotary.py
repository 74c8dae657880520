"""Rotate-half rotary position encoding.

The table of cos and sin of `pos * theta^(-2j/rot)` is built on the host in
float64 and kept in fp32, as the reference builds it
(`src/core_kernels/rope_table.cu:18-31`, `rope_angle.cuh:15-21`); the kernel
rotates in fp32 (`csrc/rope.cu`). Queries are rotated in place; keys are rotated
on their way into the cache, in the same launch that stores the values.
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import Part, register_part


class RotaryHalf(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and in "
                             f"(0, head_dim {spec.head_dim}]")
        self.cos = self.sin = None

    def prepare(self, device, max_positions):
        n = min(max_positions, self.spec.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n and self.cos.device == torch.device(device):
            return
        rot = self.spec.rotary_dim
        j = np.arange(rot // 2, dtype=np.float64)
        inv_freq = np.power(float(self.spec.theta), -2.0 * j / rot)
        angle = np.arange(n, dtype=np.float64)[:, None] * inv_freq[None, :]
        self.cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(device)
        self.sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(device)

    def tables(self, step, head_dim):
        """(cos, sin) for a kernel that rotates on its own way (the decode attention), or None
        if this encoding is not a rotation over the whole head of positions the tables hold."""
        if self.spec.rotary_dim != head_dim or self.cos.dtype != torch.float32 \
                or step.max_position >= self.cos.shape[0]:
            return None
        return self.cos, self.sin

    def rotate_store(self, qkv, step, view, heads, kv_heads, head_dim, write_cache=True):
        if step.max_position >= self.cos.shape[0]:
            raise ValueError(f"position {step.max_position} is beyond the rotary table of "
                             f"{self.cos.shape[0]} positions")
        ops.rope_store(qkv, step.positions, step.token_seq, view.block_table, self.cos, self.sin,
                       view.keys, view.values, heads, kv_heads, head_dim, write_cache)


class NoPosition(Part):
    """No position encoding: keys and values go to the cache as they are."""

    def rotate_store(self, qkv, step, view, heads, kv_heads, head_dim, write_cache=True):
        ops.rope_store(qkv, step.positions, step.token_seq, view.block_table, None, None,
                       view.keys, view.values, heads, kv_heads, head_dim, write_cache)


register_part("rotary_half", RotaryHalf)
register_part("no_position", NoPosition)

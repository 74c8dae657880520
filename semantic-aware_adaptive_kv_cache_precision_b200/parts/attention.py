"""Grouped-query causal self-attention over the cache.

    q, k, v = split(h Wqkv^T + bqkv);  q, k = position(q, k);  cache <- k, v
    out = softmax(q k^T * scale + mask) v;  residual += out Wo^T (+ bo)

as the reference runs it (`src/microinfer/model.py:375-387`), except that the
three projections are one product over the rows [Wq; Wk; Wv] laid back to back
in device memory, and that the key's bias goes through the projection and the
rotation with the key (the reference adds it, rotated, inside attention, which
is the same sum; `src/core_kernels/attention.cu:104-116`). The mask lets a
query at position p see keys j <= p, and only those with p - j < window where
the spec has a window. Sizes, scale, window and whether there are biases come
from the spec.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.needs import KVNeed
from ..weights.decl import TensorDecl
from .base import Part, build_part, register_part


class GQAAttention(Part):
    def __init__(self, spec, prefix, mode):
        super().__init__(spec, prefix, mode)
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError(f"{s.heads} heads are not a multiple of {s.kv_heads} kv heads")
        if s.head_dim % 16 or s.head_dim > 256:
            raise ValueError(f"head_dim {s.head_dim}: the attention kernels take multiples "
                             "of 16 up to 256")
        self.position = build_part(s.position, prefix, mode) if s.position is not None \
            else build_part(_NO_POSITION, prefix, mode)

    # -- tensors --------------------------------------------------------------

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        q, kv = s.heads * s.head_dim, s.kv_heads * s.head_dim
        decls = []
        for name, rows in (("q_proj", q), ("k_proj", kv), ("v_proj", kv)):
            decls.append(TensorDecl(f"{p}{name}.weight", (rows, s.hidden), group=p + "qkv.weight"))
        if s.qkv_bias:
            for name, rows in (("q_proj", q), ("k_proj", kv), ("v_proj", kv)):
                decls.append(TensorDecl(f"{p}{name}.bias", (rows,), group=p + "qkv.bias"))
        decls.append(TensorDecl(f"{p}o_proj.weight", (s.hidden, q)))
        if s.out_bias:
            decls.append(TensorDecl(f"{p}o_proj.bias", (s.hidden,)))
        return decls + self.position.tensor_decls()       # a learned position table, if any

    def bind(self, arena):
        p = self.prefix
        names = ("q_proj", "k_proj", "v_proj")
        self.w_qkv = arena.group_view(p + "qkv.weight")
        if self.w_qkv is None:
            self.w_qkv = torch.cat([arena.view(f"{p}{n}.weight") for n in names])
        self.b_qkv = None
        if self.spec.qkv_bias:
            self.b_qkv = arena.group_view(p + "qkv.bias")
            if self.b_qkv is None:
                self.b_qkv = torch.cat([arena.view(f"{p}{n}.bias") for n in names])
        self.w_o = arena.view(p + "o_proj.weight")
        self.b_o = arena.view(p + "o_proj.bias") if self.spec.out_bias else None
        self.position.bind(arena)

    def prepare(self, device, max_positions):
        self.position.prepare(device, max_positions)

    # -- cache ----------------------------------------------------------------

    def cache_need(self):
        return KVNeed(self.spec.kv_heads, self.spec.head_dim, self.spec.window)

    # -- the step ---------------------------------------------------------------

    can_defer = True

    def forward(self, h, step, view, residual, write_cache=True, defer=False):
        s = self.spec
        qkv = ops.linear(h, self.w_qkv, self.b_qkv, out_dtype=self.act_dtype)
        rotary = None
        if step.is_decode and ops.fast_path_takes(qkv.dtype, s.heads, s.kv_heads, s.head_dim) \
                and hasattr(self.position, "tables"):
            # one token a sequence: the attention kernel rotates and stores on its own way
            rotary = self.position.tables(step, s.head_dim)
        if rotary is None:
            self.position.rotate_store(qkv, step, view, s.heads, s.kv_heads, s.head_dim,
                                       write_cache)
        attended = self.attend(qkv, step, view, rotary, write_cache)
        out = ops.linear(attended, self.w_o, self.b_o, accumulate_into=residual, may_defer=defer)
        return out.delta if isinstance(out, ops.Deferred) else None

    def attend(self, qkv, step, view, rotary=None, write_cache=True):
        """Tensor-core kernels where they take the sizes (bf16, head_dim 64 or 128, up
        to 16 query heads per KV head): the split-key decode kernel when every
        sequence brings one token; otherwise the causal prefill kernels, tcgen05 for
        head size 128 and mma.sync for 64. Everything else, and the whole fp32 path,
        runs the plain kernel."""
        s = self.spec
        if ops.fast_path_takes(qkv.dtype, s.heads, s.kv_heads, s.head_dim):
            if step.is_decode:
                return ops.attention_decode(qkv, view.keys, view.values, step.seq_lens,
                                            view.block_table, s.heads, s.kv_heads, s.head_dim,
                                            s.scale, s.window, step.max_len_bound or step.max_len,
                                            rotary=rotary, write_cache=write_cache)
            if ops.tc_prefill_takes(qkv.dtype, s.heads, s.kv_heads, s.head_dim) and step.starts:
                key = ("wide_tiles", s.heads, s.window)
                plan = step.plans.get(key)
                if plan is None:       # the same for every layer of these sizes: made once a step
                    plan = step.plans[key] = ops.upload_wide_plan(
                        step.starts, step.new_counts, s.heads, s.window, qkv.device)
                return ops.attention_prefill_tc(qkv, view.keys, view.values, *plan,
                                                step.seq_lens, view.block_table, s.heads,
                                                s.kv_heads, s.head_dim, s.scale, s.window)
            tiles = step.plans.get("query_tiles_64")
            if tiles is None:          # the same for every attention layer: made once a step
                tiles = step.plans["query_tiles_64"] = ops.upload_query_tiles(
                    step.starts, step.new_counts, qkv.device)
            return ops.attention_prefill(qkv, view.keys, view.values, tiles,
                                         step.seq_lens, view.block_table, s.heads, s.kv_heads,
                                         s.head_dim, s.scale, s.window)
        return ops.attention_plain(qkv, view.keys, view.values, step.positions, step.token_seq,
                                   view.block_table, s.heads, s.kv_heads, s.head_dim, s.scale,
                                   s.window)


class _NoPositionSpec:
    kind = "no_position"


_NO_POSITION = _NoPositionSpec()

register_part("gqa_attention", GQAAttention)

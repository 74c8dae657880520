"""The kernels as Python functions over torch tensors.

Each function checks devices, types, shapes and strides, then launches on the
current CUDA stream. Nothing here computes on the host, and there is no other
implementation behind these functions: on a machine without the compiled
kernels they raise.
"""

from __future__ import annotations

import torch

from ._lib import (BF16, CACHE_BLOCK, F32, KernelError, call, dtype_code, plain_function, ptr,
                   require_cuda)
from .linear import Deferred, gated_up, linear
from . import gemm_tc
from .attention import (attention_decode, attention_prefill, attention_prefill_tc, decode_splits,
                        forget_descriptors,
                        fast_path_takes, kernel_errors, plan_wide_tiles, tc_prefill_takes, upload_query_tiles,
                        upload_wide_plan)

__all__ = ["CACHE_BLOCK", "KernelError", "embed", "rms_norm", "rope_store", "attention_plain",
           "attention_decode", "attention_prefill", "attention_prefill_tc", "tc_prefill_takes", "plan_wide_tiles", "upload_wide_plan",
           "upload_query_tiles",
           "decode_splits", "fast_path_takes", "forget_descriptors",
           "kernel_errors", "gated_silu", "gated_up", "gemm_tc", "add_into", "scale_cap_", "linear", "choose", "Deferred"]


def _check(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 rows of `table` for int32 `ids`; an id outside the table gives zeros."""
    require_cuda(ids, table)
    _check(ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(), "ids: int32 [T]")
    _check(table.dim() == 2 and table.is_contiguous(), "table: contiguous [vocab, hidden]")
    vocab, hidden = table.shape
    if out is None:
        out = torch.empty((ids.numel(), hidden), dtype=torch.float32, device=ids.device)
    _check(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (ids.numel(), hidden),
           "out: fp32 [T, hidden]")
    call("sakv_embed", ptr(ids), ptr(table), dtype_code(table.dtype), ptr(out), ids.numel(),
         hidden, vocab)
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
             rows: torch.Tensor | None = None, add: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of rows of fp32 `x`; with `rows` (int32), of those rows only. With `add`
    (fp32, x's shape or [parts, *x's shape]; bf16 weight and output) `x += add` (`+=
    add.sum(0)`, in order) happens first, in the same kernel, and x keeps the sum."""
    require_cuda(x, weight, rows, add)
    _check(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x: fp32 [T, hidden]")
    hidden = x.shape[1]
    _check(weight.shape == (hidden,) and weight.is_contiguous(), "weight: [hidden]")
    n = x.shape[0]
    if rows is not None:
        _check(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(),
               "rows: int32 [R]")
        n = rows.numel()
    if add is not None:
        _check(rows is None and add.dtype == torch.float32 and add.is_contiguous()
               and (add.shape == x.shape or (add.dim() == 3 and add.shape[1:] == x.shape))
               and weight.dtype == torch.bfloat16 and out_dtype == torch.bfloat16,
               "add: fp32 like x or [parts, *x.shape], bf16 weight and output, no rows")
    parts = add.shape[0] if add is not None and add.dim() == 3 else 1
    out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    call("sakv_rmsnorm", ptr(x), ptr(add), parts, x.numel(), ptr(rows), ptr(weight), dtype_code(weight.dtype), ptr(out),
         dtype_code(out_dtype), n, hidden, float(eps))
    return out


def rope_store(qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
               block_table: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None,
               k_cache: torch.Tensor | None, v_cache: torch.Tensor | None, heads: int,
               kv_heads: int, head_dim: int, write_cache: bool = True) -> None:
    """Rotate the queries of `qkv` in place; rotate the keys and write them and the
    values into the cache entry `k_cache`/`v_cache` ([blocks, kv_heads, 64, head_dim])."""
    require_cuda(qkv, positions, token_seq, block_table, cos, sin, k_cache, v_cache)
    tokens = qkv.shape[0]
    _check(qkv.dim() == 2 and qkv.stride(1) == 1
           and qkv.shape[1] == (heads + 2 * kv_heads) * head_dim,
           "qkv: [T, (heads + 2 kv_heads) head_dim]")
    for t, name in ((positions, "positions"), (token_seq, "token_seq")):
        _check(t.dtype == torch.int32 and t.is_contiguous() and t.numel() == tokens,
               f"{name}: int32 [T]")
    _check(block_table.dtype == torch.int32 and block_table.dim() == 2
           and block_table.is_contiguous(), "block_table: int32 [B, max_blocks]")
    rot = 0
    if cos is not None:
        _check(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.dim() == 2
               and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape,
               "cos, sin: fp32 [positions, rot / 2]")
        rot = 2 * cos.shape[1]
    if write_cache:
        for c in (k_cache, v_cache):
            _check(c is not None and c.dtype == qkv.dtype and c.is_contiguous() and c.dim() == 4
                   and tuple(c.shape[1:]) == (kv_heads, CACHE_BLOCK, head_dim),
                   "cache entry: [blocks, kv_heads, 64, head_dim] of the activations' type")
    call("sakv_rope_store", ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0), ptr(positions),
         ptr(token_seq), ptr(block_table), block_table.shape[1], ptr(cos), ptr(sin), rot,
         ptr(k_cache), ptr(v_cache), tokens, heads, kv_heads, head_dim, int(write_cache))


def attention_plain(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor,
                    heads: int, kv_heads: int, head_dim: int, scale: float,
                    window: int | None) -> torch.Tensor:
    """Causal grouped-query attention of every token of the step over its sequence's
    cache; queries are the first heads*head_dim columns of `qkv`."""
    require_cuda(qkv, k_cache, v_cache, positions, token_seq, block_table)
    tokens = qkv.shape[0]
    _check(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= heads * head_dim,
           "qkv: [T, >= heads * head_dim]")
    _check(head_dim <= 256, f"head_dim {head_dim}: the plain attention kernel takes up to 256")
    _check(heads % kv_heads == 0, "heads must be a multiple of kv_heads")
    for c in (k_cache, v_cache):
        _check(c.dtype == qkv.dtype and c.is_contiguous() and c.dim() == 4
               and tuple(c.shape[1:]) == (kv_heads, CACHE_BLOCK, head_dim),
               "cache entry: [blocks, kv_heads, 64, head_dim] of the activations' type")
    out = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    call("sakv_attention_plain", ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0), ptr(out),
         ptr(k_cache), ptr(v_cache), ptr(positions), ptr(token_seq), ptr(block_table),
         block_table.shape[1], tokens, heads, kv_heads, head_dim, float(scale),
         int(window) if window else 0)
    return out


def gated_silu(gate_up: torch.Tensor) -> torch.Tensor:
    """`silu(gate) * up` for `gate_up[t] = [gate | up]`."""
    require_cuda(gate_up)
    _check(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0,
           "gate_up: contiguous [T, 2 * intermediate]")
    tokens, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    call("sakv_gated_silu", ptr(gate_up), ptr(out), dtype_code(gate_up.dtype), tokens, inter)
    return out


def add_into(acc: torch.Tensor, y: torch.Tensor) -> None:
    """`acc += y` with `acc` fp32; `y` of acc's shape, or [parts, *acc.shape], whose parts are
    summed first, in order (as `rms_norm(add=...)` does)."""
    require_cuda(acc, y)
    if y.dim() == acc.dim() + 1:
        total = y[0]
        if y.shape[0] > 1:
            total = y[0].clone()
            for part in y[1:]:
                add_into(total, part)
        y = total
    _check(acc.dtype == torch.float32 and acc.is_contiguous() and y.is_contiguous()
           and acc.shape == y.shape, "acc: fp32, same shape as y, both contiguous")
    call("sakv_add_into", ptr(acc), ptr(y), dtype_code(y.dtype), acc.numel())


def scale_cap_(x: torch.Tensor, scale: float = 1.0, cap: float | None = None) -> torch.Tensor:
    """In place on fp32 `x`: `x *= scale`, then with `cap` c, `x = c * tanh(x / c)`."""
    require_cuda(x)
    _check(x.dtype == torch.float32 and x.is_contiguous(), "x: contiguous fp32")
    _check(cap is None or cap > 0, "cap must be positive")
    call("sakv_scale_cap", ptr(x), x.numel(), float(scale), float(cap or 0.0))
    return x


def choose(logits: torch.Tensor, temperature: float = 0.0, seed: int = 0,
           request: torch.Tensor | None = None, step: torch.Tensor | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of fp32 `logits`: greedy at temperature 0, else a
    Gumbel-max draw keyed by (seed, request[row], step[row]). `out` (int32 [rows], contiguous):
    where to write them, instead of a new tensor."""
    require_cuda(logits, request, step, out)
    _check(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1,
           "logits: fp32 [rows, vocab]")
    rows, vocab = logits.shape
    if temperature > 0:
        for t, name in ((request, "request"), (step, "step")):
            _check(t is not None and t.dtype == torch.int32 and t.is_contiguous()
                   and t.numel() == rows, f"{name}: int32 [rows]")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        _check(out.dtype == torch.int32 and out.shape == (rows,) and out.is_contiguous(),
               "out: int32 [rows]")
    chunks = plain_function("sakv_choose_chunks")(vocab)
    scratch = _choose_scratch.get(logits.device)
    if scratch is None or scratch[0].numel() < rows * chunks or scratch[1].numel() < rows:
        scratch = (torch.empty(max(rows * chunks, 4096), dtype=torch.int64, device=logits.device),
                   torch.zeros(max(rows, 1024), dtype=torch.int32, device=logits.device))
        _choose_scratch[logits.device] = scratch
    call("sakv_choose", ptr(logits), logits.stride(0) if rows else vocab, rows, vocab,
         float(temperature), int(seed) & 0xFFFFFFFFFFFFFFFF, ptr(request), ptr(step), ptr(out),
         ptr(scratch[0]), ptr(scratch[1]))
    return out


_choose_scratch: dict = {}

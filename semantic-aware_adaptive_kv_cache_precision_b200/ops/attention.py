"""The bfloat16 tensor-core attention kernels: split-key decode and causal prefill,
both reading keys and values straight from the cache's blocks by TMA."""

from __future__ import annotations

import ctypes

import torch

from ._lib import CACHE_BLOCK, KernelError, call, plain_function, ptr, require_cuda

SM_COUNT = 148
_maps: dict = {}


def fast_path_takes(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core kernels take these sizes (else the plain kernel runs)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and heads % kv_heads == 0
            and heads // kv_heads <= 16)


def tensor_map(cache: torch.Tensor):
    """The TMA descriptor of one cache entry [blocks, kv_heads, 64, head_dim] (bf16),
    made once per tensor and kept; returns the address of its 128 bytes on the host."""
    key = (cache.data_ptr(), tuple(cache.shape))
    hit = _maps.get(key)
    if hit is None:
        if cache.dtype != torch.bfloat16 or not cache.is_contiguous() or cache.dim() != 4 \
                or cache.shape[2] != CACHE_BLOCK:
            raise KernelError("tensor_map: cache entry must be contiguous bf16 "
                              "[blocks, kv_heads, 64, head_dim]")
        raw = ctypes.create_string_buffer(128 + 64)
        address = (ctypes.addressof(raw) + 63) & ~63
        code = plain_function("sakv_decode_attention_map")(
            address, cache.data_ptr(), cache.shape[0], cache.shape[1], cache.shape[3])
        if code != 0:
            raise KernelError(f"could not make a TMA descriptor for the cache (error {code})")
        hit = (raw, address)
        _maps[key] = hit
    return hit[1]


def decode_splits(sequences: int, kv_heads: int, max_len: int) -> int:
    """How many ways to split the keys so that about one block per SM is busy."""
    tiles = max(1, -(-max_len // CACHE_BLOCK))
    pairs = max(1, sequences * kv_heads)
    want = max(1, SM_COUNT // pairs)
    if want == 1 and pairs < 2 * SM_COUNT and tiles >= 8:
        want = 2          # two blocks fit an SM: more tiles in flight (29 us against 37 at batch 64)
    return max(1, min(tiles, want, 32))


def attention_decode(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     seq_lens: torch.Tensor, block_table: torch.Tensor, heads: int, kv_heads: int,
                     head_dim: int, scale: float, window, max_len: int,
                     splits: int | None = None) -> torch.Tensor:
    """One query token per sequence (row b of `qkv` belongs to sequence b)."""
    require_cuda(qkv, k_cache, v_cache, seq_lens, block_table)
    sequences = qkv.shape[0]
    if not fast_path_takes(qkv.dtype, heads, kv_heads, head_dim):
        raise KernelError("attention_decode: sizes not taken; use the plain kernel")
    if qkv.stride(1) != 1 or qkv.shape[1] < heads * head_dim or (qkv.stride(0) % 2):
        raise KernelError("attention_decode: qkv must be [B, >= heads * head_dim], rows contiguous")
    if seq_lens.numel() != sequences or block_table.shape[0] != sequences:
        raise KernelError("attention_decode: one length and one block list per sequence")
    if splits is None:
        splits = decode_splits(sequences, kv_heads, max_len)
    out = torch.empty((sequences, heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((sequences, heads, splits, head_dim), dtype=torch.float32,
                             device=qkv.device)
        part_ml = torch.empty((sequences, heads, splits, 2), dtype=torch.float32,
                              device=qkv.device)
    call("sakv_decode_attention", tensor_map(k_cache), tensor_map(v_cache), ptr(qkv),
         qkv.stride(0), ptr(seq_lens), ptr(block_table), block_table.shape[1], ptr(out),
         ptr(part_o), ptr(part_ml), sequences, heads, kv_heads, head_dim, splits, float(scale),
         int(window) if window else 0)
    return out


def attention_prefill(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      q_tiles: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
                      heads: int, kv_heads: int, head_dim: int, scale: float,
                      window) -> torch.Tensor:
    """`q_tiles`: int32 [n, 4] = (sequence, first token row, rows <= 64, first position)."""
    require_cuda(qkv, k_cache, v_cache, q_tiles, seq_lens, block_table)
    if not fast_path_takes(qkv.dtype, heads, kv_heads, head_dim):
        raise KernelError("attention_prefill: sizes not taken; use the plain kernel")
    if qkv.stride(1) != 1 or qkv.shape[1] < heads * head_dim or (qkv.stride(0) % 2):
        raise KernelError("attention_prefill: qkv must be [T, >= heads * head_dim], rows contiguous")
    if q_tiles.dtype != torch.int32 or q_tiles.dim() != 2 or q_tiles.shape[1] != 4 \
            or not q_tiles.is_contiguous():
        raise KernelError("attention_prefill: q_tiles must be int32 [n, 4]")
    out = torch.empty((qkv.shape[0], heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    call("sakv_prefill_attention", tensor_map(k_cache), tensor_map(v_cache), ptr(qkv),
         qkv.stride(0), ptr(out), ptr(q_tiles), q_tiles.shape[0], ptr(seq_lens),
         ptr(block_table), block_table.shape[1], heads, kv_heads, head_dim, float(scale),
         int(window) if window else 0)
    return out


def tc_prefill_takes(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tcgen05 prefill kernel takes these sizes (head size 128)."""
    return dtype == torch.bfloat16 and head_dim == 128 and heads % kv_heads == 0


def attention_prefill_tc(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         q_tiles: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
                         heads: int, kv_heads: int, head_dim: int, scale: float,
                         window) -> torch.Tensor:
    """The tcgen05 prefill kernel. `q_tiles`: int32 [n, 4] = (sequence, first token row,
    rows <= 128, first position)."""
    require_cuda(qkv, k_cache, v_cache, q_tiles, seq_lens, block_table)
    if not tc_prefill_takes(qkv.dtype, heads, kv_heads, head_dim):
        raise KernelError("attention_prefill_tc: sizes not taken (bf16, head_dim 128)")
    if qkv.stride(1) != 1 or qkv.shape[1] < heads * head_dim or (qkv.stride(0) % 8) \
            or qkv.data_ptr() % 16:
        raise KernelError("attention_prefill_tc: qkv must be [T, >= heads * head_dim] with rows "
                          "a multiple of 16 bytes apart")
    if q_tiles.dtype != torch.int32 or q_tiles.dim() != 2 or q_tiles.shape[1] != 4 \
            or not q_tiles.is_contiguous():
        raise KernelError("attention_prefill_tc: q_tiles must be int32 [n, 4]")
    raw = ctypes.create_string_buffer(128 + 64)
    q_map = (ctypes.addressof(raw) + 63) & ~63
    code = plain_function("sakv_prefill_attention_tc_qmap")(q_map, qkv.data_ptr(), qkv.shape[0],
                                                            qkv.shape[1], qkv.stride(0))
    if code != 0:
        raise KernelError(f"could not make a TMA descriptor for the queries (error {code})")
    out = torch.empty((qkv.shape[0], heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    call("sakv_prefill_attention_tc", q_map, tensor_map(k_cache), tensor_map(v_cache), ptr(out),
         ptr(q_tiles), q_tiles.shape[0], ptr(seq_lens), ptr(block_table), block_table.shape[1],
         heads, kv_heads, head_dim, float(scale), int(window) if window else 0)
    return out


def kernel_errors() -> dict:
    """Error words left by waits that gave up (0 = none). Synchronises the device."""
    out = {}
    for name in ("sakv_decode_attention_error", "sakv_prefill_attention_error",
                 "sakv_prefill_attention_tc_error"):
        value = ctypes.c_int(0)
        code = plain_function(name)(ctypes.addressof(value))
        out[name] = value.value if code == 0 else -code
    return out

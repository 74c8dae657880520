"""The bfloat16 tensor-core attention kernels: split-key decode and causal prefill,
both reading keys and values straight from the cache's blocks by TMA."""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import CACHE_BLOCK, KernelError, call, plain_function, ptr, require_cuda, sm_count

_maps: dict = {}


def fast_path_takes(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core kernels take these sizes (else the plain kernel runs)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and heads % kv_heads == 0
            and heads // kv_heads <= 16)


def tensor_map(cache: torch.Tensor):
    """The TMA descriptor of one cache entry [blocks, kv_heads, 64, head_dim] (bf16),
    made once per tensor and kept; returns the address of its 128 bytes on the host."""
    key = (cache.data_ptr(), tuple(cache.shape), cache.stride(), cache.dtype)
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


# The numbers of splits whose blocks fold their partials themselves, as one thread-block
# cluster, instead of leaving them to a second kernel. Measured inside the decode step at the
# 1.5B widths, 2,048 cached tokens (ms a step, second kernel / cluster): 64 sequences (2
# splits) 2.09 / 2.06, 32 (4) 1.59 / 1.53; but 48 (3) 1.86 / 2.10, 24 (6) 1.47 / 1.58, 16 (9)
# 1.34 / 1.47, 12 (11) 1.31 / 1.45, 8 (9) 1.216 / 1.218, 8 (8) 1.222, 4 (16) 1.20 against 1.15
# with 18 splits: clusters of 2 and 4 find their SMs at once, the others wait for a placement.
FOLD_IN_CLUSTER = (2, 4)

_fold_limit: dict = {}


def fold_cluster_limit(head_dim: int) -> int:
    """How many splits the decode kernel folds by itself, as one thread-block cluster (asked of
    the device once: 16 where non-portable cluster sizes are granted, else 8)."""
    key = (head_dim, torch.cuda.current_device())
    if key not in _fold_limit:
        _fold_limit[key] = int(plain_function("sakv_decode_attention_max_cluster")(head_dim))
    return _fold_limit[key]


def decode_splits(sequences: int, kv_heads: int, max_len: int, sms: int | None = None) -> int:
    """How many ways to split the keys. Either one block per SM, however short its run of
    keys, or, when that leaves runs of many tiles, two blocks per SM with at least three
    tiles each: more tiles in flight. Measured at 2,053 keys, 2 KV heads (us, fold included):
    8 sequences 9 splits 8.1 (12: 8.7); 16 sequences 4: 12.6, 9: 10.5; 32 sequences 2: 22.9,
    4: 16.1; 64 sequences 1: 35.5, 2: 28.3."""
    sms = sms or sm_count()
    tiles = max(1, -(-max_len // CACHE_BLOCK))
    pairs = max(1, sequences * kv_heads)
    one_each = max(1, min(tiles, sms // pairs))
    two_each = max(1, min(tiles // 3, 2 * sms // pairs))
    if two_each * pairs > sms and 2 * two_each >= 3 * one_each:
        return min(two_each, 64)
    return min(one_each, 64)


def attention_decode(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     seq_lens: torch.Tensor, block_table: torch.Tensor, heads: int, kv_heads: int,
                     head_dim: int, scale: float, window, max_len: int,
                     splits: int | None = None, rotary=None, write_cache: bool = True,
                     in_cluster: bool | None = None) -> torch.Tensor:
    """One query token per sequence (row b of `qkv` belongs to sequence b).

    `rotary`: None, or `(cos, sin)` (fp32 [positions, head_dim / 2], rotation over the whole
    head): `qkv` is then the projection's output as it came, [q | k | v] unrotated, and the
    kernel rotates the queries on its way and (`write_cache`) puts the newest position's
    rotated key and its value into the cache; `ops.rope_store` is not called for the step."""
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
    if in_cluster is None:      # (a device that places no such cluster: the second kernel)
        in_cluster = splits in FOLD_IN_CLUSTER and splits <= fold_cluster_limit(head_dim)
    if in_cluster and not 1 < splits <= fold_cluster_limit(head_dim):
        if splits > 1:
            raise KernelError(f"attention_decode: {splits} splits do not fold as one cluster "
                              f"(at most {fold_cluster_limit(head_dim)})")
        in_cluster = False
    out = torch.empty((sequences, heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    part_o = part_ml = None
    if splits > 1 and not in_cluster:
        part_o = torch.empty((sequences, heads, splits, head_dim), dtype=torch.float32,
                             device=qkv.device)
        part_ml = torch.empty((sequences, heads, splits, 2), dtype=torch.float32,
                              device=qkv.device)
    call("sakv_decode_attention", tensor_map(k_cache), tensor_map(v_cache), ptr(qkv),
         qkv.stride(0), ptr(seq_lens), ptr(block_table), block_table.shape[1], ptr(out),
         ptr(part_o), ptr(part_ml), sequences, heads, kv_heads, head_dim, splits, float(scale),
         int(window) if window else 0, *_rotary_arguments(rotary, write_cache, qkv, k_cache, v_cache,
                                                         heads, kv_heads, head_dim, max_len))
    if part_o is not None:
        _lib.launches += 1          # the call launched the fold kernel too
    return out


def _rotary_arguments(rotary, write_cache, qkv, k_cache, v_cache, heads, kv_heads, head_dim,
                      max_len):
    if rotary is None:
        return None, None, 0, None, None
    cos, sin = rotary
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != sin.shape \
            or cos.dim() != 2 or cos.shape[1] * 2 != head_dim or not cos.is_contiguous() \
            or not sin.is_contiguous():
        raise KernelError("attention_decode: rotary tables must be fp32 [positions, head_dim / 2]")
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim or qkv.data_ptr() % 16 \
            or qkv.stride(0) % 8:
        raise KernelError("attention_decode: with rotary tables qkv must be the whole "
                          "[q | k | v] projection, rows 16-byte aligned")
    if write_cache:
        return ptr(cos), ptr(sin), cos.shape[0], ptr(k_cache), ptr(v_cache)
    return ptr(cos), ptr(sin), cos.shape[0], None, None


def upload_query_tiles(starts, counts, device, tile: int = 64) -> torch.Tensor:
    """The launch plan of `attention_prefill` for sequences that hold `starts[i]` positions
    and bring `counts[i]` tokens: int32 [n, 4] on the device, one row (sequence, first token
    row, rows <= 64, first position) per query tile, none crossing a sequence's end, the
    tiles with the most keys first."""
    tiles, row = [], 0
    for i, (s, c) in enumerate(zip(starts, counts)):
        for a in range(0, c, tile):
            tiles.append((i, row + a, min(tile, c - a), s + a))
        row += c
    tiles.sort(key=lambda t: -(t[3] + t[2]))
    flat = torch.tensor(tiles, dtype=torch.int32).reshape(-1, 4)
    return flat.pin_memory().to(device, non_blocking=True)


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


def plan_wide_tiles(starts, counts, heads: int, window=None, tile: int = 128,
                    slots: int | None = None):
    """Work items and folds of the tcgen05 prefill kernel for sequences that hold `starts[i]`
    positions and bring `counts[i]` tokens. Each query tile of up to 128 tokens walks the key
    tiles (64 keys) its rows can see. When all blocks of the step run at once (`slots` of
    them fit the GPU), the longest tile decides its time, so the key tiles of the long ones
    are dealt to several blocks that leave partials to be folded; with more blocks than that
    the fold costs more than the balance gains (measured: 2,048 tokens 46 -> 38 us, 4,096
    tokens 92 -> 98 us). Returns (work [n, 8], folds [m, 4], partials)."""
    if slots is None:
        slots = 2 * sm_count()                   # two blocks of the kernel fit an SM
    tiles, row = [], 0
    for i, (s, c) in enumerate(zip(starts, counts)):
        for a in range(0, c, tile):
            rows, pos0 = min(tile, c - a), s + a
            last = pos0 + rows - 1
            first_key = max(0, pos0 - window + 1) if window else 0
            t0 = first_key // CACHE_BLOCK
            tiles.append((i, row + a, rows, pos0, t0, last // CACHE_BLOCK + 1 - t0))
        row += c
    steps = sum(t[5] for t in tiles) * heads
    limit = None
    if len(tiles) * heads < slots:                         # one wave: balance it
        limit = max(8, -(-steps * 13 // (slots * 10)))
        # ... and keep it one wave: the pieces must not outnumber the blocks that run at once
        # (2,048 tokens, 12 heads: a limit of 15 gave 312 blocks for 296 places, and the 16
        # that had to wait cost the prefill 0.05 ms of 5.50)
        while sum(1 if t[5] <= limit else -(-t[5] // limit) for t in tiles) * heads > slots:
            limit += 1
    work, folds, partials = [], [], 0
    for (i, r0, rows, pos0, t0, n) in tiles:
        pieces = 1 if limit is None or n <= limit else -(-n // limit)
        if pieces == 1:
            work.append((i, r0, rows, pos0, t0, n, -1, 0))
            continue
        per = -(-n // pieces)
        folds.append((partials, pieces, r0, rows))
        for p in range(pieces):
            work.append((i, r0, rows, pos0, t0 + p * per, min(per, n - p * per), partials, 0))
            partials += 1
    work.sort(key=lambda w: -w[5])                         # the longest blocks start first
    return work, folds, partials


def upload_wide_plan(starts, counts, heads: int, window, device, **how):
    """`plan_wide_tiles` on the device: (work, folds or None, partials)."""
    work, folds, partials = plan_wide_tiles(starts, counts, heads, window, **how)
    flat = torch.tensor([x for w in work for x in w] + [x for f in folds for x in f],
                        dtype=torch.int32).pin_memory().to(device, non_blocking=True)
    n = 8 * len(work)
    return (flat[:n].view(-1, 8), flat[n:].view(-1, 4) if folds else None, partials)


_wide_scratch: dict = {}


def attention_prefill_tc(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         work: torch.Tensor, folds, partials: int, seq_lens: torch.Tensor,
                         block_table: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                         scale: float, window) -> torch.Tensor:
    """The tcgen05 prefill kernel. `work` (int32 [n, 8]), `folds` (int32 [m, 4] or None) and
    `partials` come from `plan_wide_tiles`, on the device."""
    require_cuda(qkv, k_cache, v_cache, work, seq_lens, block_table)
    if not tc_prefill_takes(qkv.dtype, heads, kv_heads, head_dim):
        raise KernelError("attention_prefill_tc: sizes not taken (bf16, head_dim 128)")
    if qkv.stride(1) != 1 or qkv.shape[1] < heads * head_dim or (qkv.stride(0) % 8) \
            or qkv.data_ptr() % 16:
        raise KernelError("attention_prefill_tc: qkv must be [T, >= heads * head_dim] with rows "
                          "a multiple of 16 bytes apart")
    if work.dtype != torch.int32 or work.dim() != 2 or work.shape[1] != 8 \
            or not work.is_contiguous():
        raise KernelError("attention_prefill_tc: work must be int32 [n, 8]")
    raw = ctypes.create_string_buffer(128 + 64)
    q_map = (ctypes.addressof(raw) + 63) & ~63
    code = plain_function("sakv_prefill_attention_tc_qmap")(q_map, qkv.data_ptr(), qkv.shape[0],
                                                            qkv.shape[1], qkv.stride(0))
    if code != 0:
        raise KernelError(f"could not make a TMA descriptor for the queries (error {code})")
    out = torch.empty((qkv.shape[0], heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    part_o = part_ml = None
    n_folds = 0 if folds is None else folds.shape[0]
    if n_folds:
        need = partials * heads * 128 * (head_dim + 2)
        if torch.cuda.is_current_stream_capturing():
            # a graph keeps what it was captured with: scratch of its own, from its pool
            scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
        else:
            scratch = _wide_scratch.get(qkv.device)
            if scratch is None or scratch.numel() < need:
                scratch = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=qkv.device)
                _wide_scratch[qkv.device] = scratch
        part_o = scratch[:partials * heads * 128 * head_dim]
        part_ml = scratch[partials * heads * 128 * head_dim:need]
    call("sakv_prefill_attention_tc", q_map, tensor_map(k_cache), tensor_map(v_cache), ptr(out),
         ptr(work), work.shape[0], ptr(folds) if n_folds else None, n_folds, ptr(part_o),
         ptr(part_ml), ptr(seq_lens), ptr(block_table), block_table.shape[1], heads, kv_heads,
         head_dim, float(scale), int(window) if window else 0)
    if n_folds:
        _lib.launches += 1          # the call launched the fold kernel too
    return out


def forget_descriptors(*tensors) -> None:
    """Drop the kept TMA descriptors (of the cache and of weight matrices) that point into
    the memory of `tensors`. Whoever frees device memory that kernels of this library have
    read calls this, so that a later tensor at the same address gets a descriptor of its own
    and the tables do not grow with every model a process has loaded."""
    from . import gemm_tc, gemm_wide
    spans = [(t.data_ptr(), t.data_ptr() + t.numel() * t.element_size())
             for t in tensors if t is not None and t.numel()]
    for table in (_maps, gemm_tc._weight_maps, gemm_wide._weight_maps):
        for key in [k for k in table if any(lo <= k[0] < hi for lo, hi in spans)]:
            del table[key]


def kernel_errors() -> dict:
    """Error words left by waits that gave up (0 = none). Synchronises the device."""
    out = {}
    for name in ("sakv_decode_attention_error", "sakv_prefill_attention_error",
                 "sakv_prefill_attention_tc_error", "sakv_gemm_tc_error", "sakv_gemm_wide_error"):
        value = ctypes.c_int(0)
        code = plain_function(name)(ctypes.addressof(value))
        out[name] = value.value if code == 0 else -code
    return out

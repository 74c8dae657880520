"""Host side of the tcgen05 matrix product (`csrc/gemm_tc.cu`): TMA descriptors and the
choice of token tile and of the number of K splits (blocks per cluster)."""

from __future__ import annotations

import ctypes

import torch

from ._lib import BF16, F32, KernelError, call, dtype_code, plain_function, ptr, sm_count

EPI_BF16, EPI_F32, EPI_ACCUM, EPI_GATED = 0, 1, 2, 3

_weight_maps: dict = {}
MAX_PARTS = 16      # K ranges whose sums the reader adds
MAX_SPLITS = 8                # blocks of one cluster


def takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes these operands: bf16, K-major rows whose
    strides are multiples of 16 bytes, 16-byte aligned bases."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and weight.dim() == 2 and x.shape[1] == weight.shape[1] and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and x.shape[0] > 0)


def _make_map(t: torch.Tensor, box_rows: int):
    raw = ctypes.create_string_buffer(128 + 64)
    address = (ctypes.addressof(raw) + 63) & ~63
    code = plain_function("sakv_gemm_tc_map")(address, t.data_ptr(), t.shape[0], t.shape[1],
                                              t.stride(0), box_rows)
    if code != 0:
        raise KernelError(f"could not make a TMA descriptor for a {tuple(t.shape)} matrix "
                          f"(error {code})")
    return raw, address


def _weight_map(weight: torch.Tensor) -> int:
    key = (weight.data_ptr(), tuple(weight.shape), weight.stride(), weight.dtype)
    hit = _weight_maps.get(key)
    if hit is None:
        hit = _make_map(weight, 128)
        _weight_maps[key] = hit
    return hit[1]


def token_tile(m: int, dual: bool) -> int:
    for mt in (16, 32, 64, 128):
        if m <= mt:
            return mt
    return 128 if dual else 256


_cluster_room: dict = {}


def _blocks_at_once(mt: int, dual: bool, splits: int) -> int:
    """How many blocks the GPU holds at once when they come in clusters of `splits` (a
    cluster lives inside one GPC, so large clusters leave SMs unused)."""
    key = (mt, dual, splits)
    if key not in _cluster_room:
        clusters = plain_function("sakv_gemm_tc_max_clusters")(mt, int(dual), splits)
        _cluster_room[key] = min(sm_count(), clusters * splits) if clusters > 0 else \
            (sm_count() // splits) * splits * 3 // 4
    return _cluster_room[key]


def choose_splits(n_tiles: int, m_tiles: int, k: int, mt: int = 16, dual: bool = False) -> int:
    """Split K over a cluster so that as many SMs as possible pull weights in ONE wave
    (fewer splits on a tie); no split when the tiles alone fill most of the GPU."""
    tiles = n_tiles * m_tiles
    if tiles * 4 >= sm_count() * 3:
        return 1
    best, best_blocks = 1, tiles
    for splits in range(2, MAX_SPLITS + 1):
        if plain_function("sakv_gemm_tc_splits")(k, splits) != splits:
            continue
        blocks = tiles * splits
        if blocks <= _blocks_at_once(mt, dual, splits) and blocks > best_blocks:
            best, best_blocks = splits, blocks
    return best


def choose_parts(m: int, n: int, k: int) -> tuple:
    """(parts, splits) for a product whose result may be left as the sums of `parts` K
    ranges for the reader to add, each range split over a cluster of `splits` blocks; (1, 0)
    when the product is better added where it is made. Measured at 8 tokens, N = 1536, K =
    8960: two ranges over clusters of 8 take 8.2 us against 11.1 us for one cluster of 8
    adding into the stream, and the norm that adds two sums takes 0.6 us longer; for K =
    1536 nothing is gained."""
    mt = token_tile(m, False)
    tiles = -(-n // 128) * -(-m // mt)
    steps = -(-k // 64)
    if tiles * 8 * 2 > sm_count() * 3 // 2 or steps < 64:
        return 1, 0
    per = -(-steps // 16)
    if -(-steps // per) != 16:
        return 1, 0
    return 2, 8


def gemm(x: torch.Tensor, weight: torch.Tensor, bias, epi: int, out: torch.Tensor,
         n: int, dual_offset: int = 0, splits: int | None = None, parts: int = 1) -> torch.Tensor:
    """`out` is written (EPI_BF16, EPI_F32, EPI_GATED) or added to (EPI_ACCUM); `n` is the
    number of output columns (rows of `weight`, or half of them for EPI_GATED). With
    `parts` > 1 (EPI_F32, `out` [parts, M, n]) K is cut into that many ranges whose sums are
    left apart in `out[i]`, with the bias in `out[0]`."""
    m, k = x.shape
    dual = epi == EPI_GATED
    mt = token_tile(m, dual)
    n_tiles, m_tiles = -(-n // 128), -(-m // mt)
    if parts > 1:
        splits = 1 if splits is None else splits
    elif splits is None:
        splits = choose_splits(n_tiles, m_tiles, k, mt, dual)
    if parts == 1:
        splits = plain_function("sakv_gemm_tc_splits")(k, splits)
    x_raw, x_map = _make_map(x, mt)
    call("sakv_gemm_tc", _weight_map(weight), x_map, m, n, k, mt, splits, parts, epi, dual_offset,
         ptr(bias), dtype_code(bias.dtype) if bias is not None else BF16, ptr(out),
         out.stride(-2), out.stride(0) if parts > 1 else 0)
    return out


def error_word() -> int:
    value = ctypes.c_int(0)
    code = plain_function("sakv_gemm_tc_error")(ctypes.addressof(value))
    return value.value if code == 0 else -code

"""The feed-forward's gated product for many tokens on tcgen05 (`csrc/gemm_wide.cu`): tokens
on the MMA's rows, tiles of 256 tokens x (128 gate + 128 up) rows, persistent blocks, and the
gated SiLU in the epilogue."""

from __future__ import annotations

import ctypes

import torch

from ._lib import KernelError, call, plain_function, ptr

TILE_TOKENS, TILE_ROWS = 256, 128      # a block's tile: 256 tokens x (128 gate + 128 up) rows


def worth_it(tokens: int, inter: int, sms: int | None = None) -> bool:
    """Whether the fused kernel beats the library's product followed by the activation
    kernel for `tokens` tokens. Its time goes by whole waves of tiles and whole tiles of 256
    tokens, the library's by the tokens, so it wins where both are well filled. Measured with
    cold weights, fused against library (us): 1536 -> 2 x 8960: 256 tokens 31.6 / 27.6 (70
    tiles, half a wave), 512: 33.6 / 33.8, 768: 50.0 / 44.0 (1.4 waves), 1,024: 51.2 / 56.3,
    2,048: 86.5 / 92.4; 3584 -> 2 x 18944: 256 tokens 68.6 / 84.9 (148 tiles, one wave), 384:
    98.3 / 87.0 (half-empty token tiles), 1,024: 178 / 181, 1,500: 258 / 282."""
    from ._lib import sm_count
    sms = sms or sm_count()
    token_tiles = -(-tokens // TILE_TOKENS)
    tiles = token_tiles * -(-inter // TILE_ROWS)
    waves = -(-tiles // sms)
    return tokens > 64 and tiles >= 0.85 * waves * sms and tokens >= 0.8 * token_tiles * TILE_TOKENS


def pair_worth_it(tokens: int) -> bool:
    """Whether the kernel on pairs of SMs beats the library's product followed by the
    activation kernel: where its token tiles of 256 are at least five eighths (one tile) or
    four fifths (several) full.
    Measured with cold weights, pair / single block / library (us): 1536 -> 2 x 8960: 128
    tokens 21.0 / 27.4 / 34.6, 256: 20.4 / 29.2 / 35.1, 512: 27.5 / 29.2 / 36.5, 768: 35.9 /
    47.4 / 41.6, 1,024: 44.0 / 46.9 / 51.5, 2,048: 81.7 / 87.1 / 95.2, 8,192: 298 / 337 / 438;
    3584 -> 2 x 18944: 128: 56 / 59 / 61, 256: 58 / 60 / 79, 384: 95 / 98 / 85 (token tiles
    three quarters full), 512: 100 / 101 / 103, 1,024: 184 / 192 / 202, 2,048: 377 / 416 / 453;
    5120 -> 2 x 27648: 128: 116 / 156 / 116, 384: 207 / 219 / 176, 2,048: 809 / 870 / 900.
    Inside a decode step at the 1.5B widths, whose weights come from memory every time (ms a
    step, pair / library): 96 sequences 2.505 / 2.461, 128: 2.759 / 2.740, 192: 3.885 / 3.937,
    256: 4.093 / 4.148."""
    token_tiles = -(-tokens // TILE_TOKENS)
    fill = tokens / (token_tiles * TILE_TOKENS)
    return fill >= (0.625 if token_tiles == 1 else 0.8)


_pairs: dict = {}


def resident_pairs() -> int:
    """Pairs of SMs that hold the pair kernel at one time (74 on a B200; 0: not here)."""
    device = torch.cuda.current_device()
    if device not in _pairs:
        _pairs[device] = int(plain_function("sakv_gemm_pair_resident")())
    return _pairs[device]


_weight_maps: dict = {}


def takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """bf16 operands, K-major rows a multiple of 16 bytes apart, 16-byte aligned."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and weight.dim() == 2 and x.shape[1] == weight.shape[1] and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and x.shape[0] > 0)


def _make_map(t: torch.Tensor, maker: str = "sakv_gemm_wide_map"):
    """(each kernel's library makes its own descriptors, so that only the library of the
    kernel that runs is ever built)"""
    raw = ctypes.create_string_buffer(128 + 64)
    address = (ctypes.addressof(raw) + 63) & ~63
    code = plain_function(maker)(address, t.data_ptr(), t.shape[0], t.shape[1], t.stride(0))
    if code != 0:
        raise KernelError(f"could not make a TMA descriptor for a {tuple(t.shape)} matrix "
                          f"(error {code})")
    return raw, address


def _weight_map(weight: torch.Tensor, maker: str = "sakv_gemm_wide_map") -> int:
    key = (weight.data_ptr(), tuple(weight.shape), weight.stride(), weight.dtype, maker)
    hit = _weight_maps.get(key)
    if hit is None:
        hit = _weight_maps[key] = _make_map(weight, maker)
    return hit[1]


def gated(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """`silu(x Wgate^T) * (x Wup^T)` as bf16 [T, inter] for `w_gate_up = [Wgate; Wup]`."""
    inter = w_gate_up.shape[0] // 2
    if inter % 8:
        raise KernelError("gemm_wide.gated: the intermediate size must be a multiple of 8")
    out = torch.empty((x.shape[0], inter), dtype=torch.bfloat16, device=x.device)
    x_raw, x_map = _make_map(x)
    call("sakv_gemm_wide", x_map, _weight_map(w_gate_up), x.shape[0], inter, x.shape[1], inter,
         ptr(out), out.stride(0))
    return out


def gated_pair(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """The same product on pairs of SMs (`csrc/gemm_pair.cu`, tcgen05 with `cta_group::2`)."""
    inter = w_gate_up.shape[0] // 2
    if inter % 8:
        raise KernelError("gemm_wide.gated_pair: the intermediate size must be a multiple of 8")
    out = torch.empty((x.shape[0], inter), dtype=torch.bfloat16, device=x.device)
    x_raw, x_map = _make_map(x, "sakv_gemm_pair_map")
    call("sakv_gemm_pair", x_map, _weight_map(w_gate_up, "sakv_gemm_pair_map"), x.shape[0], inter, x.shape[1], inter,
         ptr(out), out.stride(0))
    return out


def pair_error_word() -> int:
    value = ctypes.c_int(0)
    code = plain_function("sakv_gemm_pair_error")(ctypes.addressof(value))
    return value.value if code == 0 else -code


def error_word() -> int:
    value = ctypes.c_int(0)
    code = plain_function("sakv_gemm_wide_error")(ctypes.addressof(value))
    return value.value if code == 0 else -code

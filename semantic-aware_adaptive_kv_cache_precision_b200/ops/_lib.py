"""ctypes access to the compiled kernels: signatures, stream and error handling."""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
CACHE_BLOCK = 64          # tokens per cache block; csrc/common.cuh has the same constant


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


P, I, L, F, U = c_void_p, c_int, c_longlong, c_float, c_ulonglong

#: exported function -> (library, argument types); the stream is always last
SIGNATURES = {
    "sakv_embed": ("elementwise", [P, P, I, P, I, I, I, P]),
    "sakv_gated_silu": ("elementwise", [P, P, I, I, I, P]),
    "sakv_add_into": ("elementwise", [P, P, I, L, P]),
    "sakv_scale_cap": ("elementwise", [P, L, F, F, P]),
    "sakv_rmsnorm": ("norm", [P, P, I, L, P, P, I, P, I, I, I, F, P]),
    "sakv_rope_store": ("rope", [P, I, L, P, P, P, I, P, P, I, P, P, I, I, I, I, I, P]),
    "sakv_attention_plain": ("attention_plain",
                             [P, I, L, P, P, P, P, P, P, I, I, I, I, I, F, I, P]),
    "sakv_gemm_f32": ("gemm_f32", [P, L, P, P, P, L, I, I, I, I, P]),
    "sakv_choose": ("sampling", [P, L, I, I, F, U, P, P, P, P, P, P]),
    "sakv_decode_attention": ("attention_decode",
                              [P, P, P, L, P, P, I, P, P, P, I, I, I, I, I, F, I, P, P, I, P, P, P]),
    "sakv_prefill_attention": ("attention_prefill",
                               [P, P, P, L, P, P, I, P, P, I, I, I, I, F, I, P]),
    "sakv_prefill_attention_tc": ("attention_prefill_tc",
                                  [P, P, P, P, P, I, P, I, P, P, P, P, I, I, I, I, F, I, P]),
    "sakv_gemm_tc": ("gemm_tc", [P, P, I, I, I, I, I, I, I, I, P, I, P, L, L, P]),
    "sakv_gemm_wide": ("gemm_wide", [P, P, I, I, I, I, P, L, P]),
    "sakv_gemm_pair": ("gemm_pair", [P, P, I, I, I, I, P, L, P]),
    "sakv_lib_accumulate": ("gemm_lib", [P, L, P, P, L, I, I, I, P, L, P]),
}

#: functions without a stream argument: (library, argument types)
PLAIN_SIGNATURES = {
    "sakv_choose_chunks": ("sampling", [I]),
    "sakv_decode_attention_map": ("attention_decode", [P, P, L, I, I]),
    "sakv_decode_attention_error": ("attention_decode", [P]),
    "sakv_decode_attention_max_cluster": ("attention_decode", [I]),
    "sakv_prefill_attention_error": ("attention_prefill", [P]),
    "sakv_prefill_attention_tc_error": ("attention_prefill_tc", [P]),
    "sakv_prefill_attention_tc_qmap": ("attention_prefill_tc", [P, P, L, L, L]),
    "sakv_gemm_tc_map": ("gemm_tc", [P, P, L, L, L, I]),
    "sakv_gemm_wide_map": ("gemm_wide", [P, P, L, L, L]),
    "sakv_gemm_pair_map": ("gemm_pair", [P, P, L, L, L]),
    "sakv_gemm_wide_error": ("gemm_wide", [P]),
    "sakv_gemm_pair_error": ("gemm_pair", [P]),
    "sakv_gemm_pair_resident": ("gemm_pair", []),
    "sakv_gemm_tc_splits": ("gemm_tc", [I, I]),
    "sakv_gemm_tc_max_clusters": ("gemm_tc", [I, I, I]),
    "sakv_gemm_tc_error": ("gemm_tc", [P]),
}

_functions: dict[str, object] = {}


def function(name: str):
    fn = _functions.get(name)
    if fn is None:
        library, argtypes = SIGNATURES[name]
        fn = getattr(_build.load(library), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _functions[name] = fn
    return fn


def plain_function(name: str):
    fn = _functions.get(name)
    if fn is None:
        library, argtypes = PLAIN_SIGNATURES[name]
        fn = getattr(_build.load(library), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _functions[name] = fn
    return fn


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def ptr(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> int:
    """The current stream of the current device, as the integer the kernels take. (The raw
    getter costs a fraction of a microsecond; `torch.cuda.current_stream()` builds a Python
    object on every call, 15 us that a prefill step pays 150 times.)"""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of `device` (default: the current one), asked once."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("this library runs on a CUDA device only: got a tensor on "
                              f"{t.device}; there is no CPU implementation")


#: kernels of this library launched by this process (benchmarks report the count)
launches = 0


def call(name: str, *args) -> None:
    global launches
    launches += 1
    code = function(name)(*args, stream())
    if code != 0:
        raise KernelError(f"{name} failed with CUDA error {code}"
                          + (" (invalid value: a size this kernel does not take)" if code == 1 else ""))

"""`y = x W^T (+ bias)`, optionally added into an fp32 accumulator.

Which kernel runs depends on the weight's type on the device:

* float32 weight: the hand-written true 32-bit product (`csrc/gemm_f32.cu`),
  whose result for a row does not depend on the other rows of the batch.
* bfloat16 weight: a bf16 tensor-core product with fp32 accumulation and one
  rounding of the result. The reference calls cuBLAS for every projection
  (`src/core_kernels/linear.cu:85-142`); here it is cuBLAS through
  `torch.mm`/`torch.addmm` until the library's own tcgen05 kernel takes a
  shape.
"""

from __future__ import annotations

import torch

from ._lib import KernelError, call, ptr, require_cuda


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, *,
           out_dtype: torch.dtype | None = None,
           accumulate_into: torch.Tensor | None = None) -> torch.Tensor:
    """`x`: [T, K]; `weight`: [N, K] as stored in the checkpoint; `bias`: [N] or None.

    With `accumulate_into` (fp32 [T, N]) the product is added to it in fp32 and it
    is returned; otherwise a new [T, N] tensor of `out_dtype` (default: x's type).
    """
    require_cuda(x, weight, bias, accumulate_into)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise KernelError(f"linear: x {tuple(x.shape)} does not fit weight {tuple(weight.shape)}")
    if x.stride(1) != 1 or not weight.is_contiguous():
        raise KernelError("linear: x rows and the weight must be contiguous")
    tokens, k = x.shape
    n = weight.shape[0]
    if accumulate_into is not None:
        acc = accumulate_into
        if acc.dtype != torch.float32 or acc.shape != (tokens, n) or acc.stride(1) != 1:
            raise KernelError("linear: accumulate_into must be fp32 [T, N]")
    out_dtype = out_dtype or x.dtype

    if weight.dtype == torch.float32:
        xf = x if x.dtype == torch.float32 else x.float()
        bf = None if bias is None else (bias if bias.dtype == torch.float32 else bias.float())
        if accumulate_into is not None:
            call("sakv_gemm_f32", ptr(xf), xf.stride(0), ptr(weight), ptr(bf), ptr(acc),
                 acc.stride(0), tokens, n, k, 1)
            return acc
        out = torch.empty((tokens, n), dtype=torch.float32, device=x.device)
        call("sakv_gemm_f32", ptr(xf), xf.stride(0), ptr(weight), ptr(bf), ptr(out),
             out.stride(0), tokens, n, k, 0)
        return out if out_dtype == torch.float32 else out.to(out_dtype)

    if weight.dtype != torch.bfloat16:
        raise KernelError(f"linear: weight type {weight.dtype} is not supported")
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    if accumulate_into is not None:
        from . import add_into
        y = torch.mm(xb, weight.t(), out_dtype=torch.float32)
        if bias is not None:
            y += bias.float()
        add_into(acc, y)
        return acc
    if out_dtype == torch.float32:
        y = torch.mm(xb, weight.t(), out_dtype=torch.float32)
        if bias is not None:
            y += bias.float()
        return y
    if bias is not None:
        return torch.addmm(bias.to(torch.bfloat16), xb, weight.t())
    return torch.mm(xb, weight.t())

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

from . import gemm_tc, gemm_wide
from ._lib import KernelError, call, ptr, require_cuda

#: up to this many tokens the library's own tcgen05 kernel runs (weights on the MMA's rows:
#: made for decode); above it cuBLAS, whose 2-CTA kernels win once the tensor cores matter
#: (measured at 128 tokens: 4.5 / 14.8 / 88 us against 8.6 / 27.9 / 137 us for QKV, gate-up
#: and the LM head)
TC_MAX_TOKENS = 64


#: whether the library's products that complete an fp32 accumulator add into it themselves
#: (cuBLAS with beta = 1, through `csrc/gemm_lib.cu`) instead of leaving the product apart
LIBRARY_ADDS_IN_PLACE = True
_WORKSPACE_BYTES = 64 << 20
_workspaces: dict = {}


_library_state = {"checked": False, "usable": False}


def _library_adds(device) -> bool:
    """Whether the wrapper around cuBLAS could be built and loaded here (it links against the
    toolkit's libcublas). It is a library product like `torch.mm`: where it cannot be had,
    the product goes through torch and a kernel of this library adds it, and a line says so."""
    if not _library_state["checked"]:
        _library_state["checked"] = True
        try:
            from ._lib import function
            function("sakv_lib_accumulate")
            _library_state["usable"] = True
        except Exception as exc:              # no libcublas to link against, say
            import sys
            print(f"[ops] the cuBLAS wrapper is not available ({type(exc).__name__}: "
                  f"{str(exc)[:200]}); products are added by a kernel of their own", file=sys.stderr)
    return _library_state["usable"]


def _library_workspace(device) -> torch.Tensor:
    space = _workspaces.get(device)
    if space is None:
        space = _workspaces[device] = torch.empty(_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
    return space


class Deferred:
    """An fp32 product that its caller still has to add to the accumulator it named."""

    __slots__ = ("delta",)

    def __init__(self, delta: torch.Tensor):
        self.delta = delta


def gated_up(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """`silu(x Wgate^T) * (x Wup^T)` for `w_gate_up = [Wgate; Wup]`: one kernel with the
    activation in its epilogue where the tensor-core kernel takes the operands, else the
    product followed by the activation kernel."""
    from . import gated_silu
    inter = w_gate_up.shape[0] // 2
    if x.shape[0] <= TC_MAX_TOKENS and inter % 128 == 0 and gemm_tc.takes(x, w_gate_up):
        out = torch.empty((x.shape[0], inter), dtype=torch.bfloat16, device=x.device)
        return gemm_tc.gemm(x, w_gate_up, None, gemm_tc.EPI_GATED, out, inter, dual_offset=inter)
    if inter % 8 == 0 and gemm_wide.takes(x, w_gate_up):
        if gemm_wide.pair_worth_it(x.shape[0]) and gemm_wide.resident_pairs() > 0:
            return gemm_wide.gated_pair(x, w_gate_up)
        if gemm_wide.worth_it(x.shape[0], inter):
            return gemm_wide.gated(x, w_gate_up)
    return gated_silu(linear(x, w_gate_up, out_dtype=x.dtype))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, *,
           out_dtype: torch.dtype | None = None,
           accumulate_into: torch.Tensor | None = None, may_defer: bool = False):
    """`x`: [T, K]; `weight`: [N, K] as stored in the checkpoint; `bias`: [N] or None.

    With `accumulate_into` (fp32 [T, N]) the product is added to it in fp32 and it
    is returned; otherwise a new [T, N] tensor of `out_dtype` (default: x's type).

    With `may_defer` as well, a product that lies in a tensor of its own is not added: the
    call returns `Deferred(delta)` with the fp32 product [T, N], or with the sums of several K
    ranges [parts, T, N], and the caller owes `accumulate_into += delta` (`+= delta.sum(0)`);
    the norm that reads the sum next can do it on its way, `rms_norm(..., add=delta)`.
    Kernels that add in their epilogue return the accumulator.
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
    if tokens <= TC_MAX_TOKENS and gemm_tc.takes(xb, weight) and \
            (bias is None or bias.dtype in (torch.bfloat16, torch.float32)):
        if accumulate_into is not None:
            parts, splits = gemm_tc.choose_parts(tokens, n, k) \
                if may_defer and acc.is_contiguous() else (1, 0)
            if parts > 1:      # few row tiles, long K: ranges summed apart, added by the reader
                sums = torch.empty((parts, tokens, n), dtype=torch.float32, device=x.device)
                return Deferred(gemm_tc.gemm(xb, weight, bias, gemm_tc.EPI_F32, sums, n,
                                             splits=splits, parts=parts))
            return gemm_tc.gemm(xb, weight, bias, gemm_tc.EPI_ACCUM, acc, n)
        if out_dtype == torch.float32:
            out = torch.empty((tokens, n), dtype=torch.float32, device=x.device)
            return gemm_tc.gemm(xb, weight, bias, gemm_tc.EPI_F32, out, n)
        if out_dtype == torch.bfloat16:
            out = torch.empty((tokens, n), dtype=torch.bfloat16, device=x.device)
            return gemm_tc.gemm(xb, weight, bias, gemm_tc.EPI_BF16, out, n)
    if accumulate_into is not None and bias is None and LIBRARY_ADDS_IN_PLACE \
            and xb.stride(1) == 1 and acc.stride(1) == 1 and _library_adds(x.device):
        # the library adds into the stream itself (beta = 1), as the reference's products do
        call("sakv_lib_accumulate", ptr(xb), xb.stride(0), ptr(weight), ptr(acc), acc.stride(0),
             tokens, n, k, ptr(_library_workspace(x.device)), _WORKSPACE_BYTES)
        return acc
    if accumulate_into is not None:
        from . import add_into
        y = torch.mm(xb, weight.t(), out_dtype=torch.float32)
        if bias is not None:
            y += bias.float()
        if may_defer and acc.is_contiguous():
            return Deferred(y)
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

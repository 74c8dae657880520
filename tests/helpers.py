"""Shared by the GPU tests: tolerances and the comparison with the plain model.

Tolerances are fixed here from the arithmetic, not from what a run happened to
give. fp32 has a unit roundoff of 2^-24; a logit is the end of a chain of a few
dozen fp32 reductions over at most a few hundred terms of size O(1), so errors
stay below 1e-5 of the logits' scale. bf16 rounds to 2^-9 relative at about ten
places per layer; over a few layers that is about 1 % of the scale of the
activations it rounds, and 6 % is the bound used (3 sigma with margin).
"""

from __future__ import annotations

import numpy as np

import plain_model as plain

FP32_RTOL = 2e-5       # of the largest |logit| of the row
BF16_RTOL = 6e-2       # of the standard deviation of the row's logits


def plain_logits(folder, ids):
    config, tensors = plain.read_model_folder(folder)
    return plain.forward(config, tensors, ids)


def assert_close_to_plain(got: np.ndarray, want: np.ndarray, dtype: str, what: str = "") -> None:
    """`got` [rows, vocab] from the engine against float64 `want`."""
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: the engine's logits are not finite"
    diff = np.abs(got.astype(np.float64) - want)
    if dtype == "float32":
        bound = FP32_RTOL * np.abs(want).max(axis=-1, keepdims=True)
    else:
        bound = BF16_RTOL * want.std(axis=-1, keepdims=True)
    worst = np.unravel_index(np.argmax(diff - bound), diff.shape)
    assert (diff <= bound).all(), (
        f"{what}: row {worst[0]} column {worst[1]} differs by {diff[worst]:.3e} "
        f"(bound {bound[worst[0], 0]:.3e}); first bad row {np.flatnonzero((diff > bound).any(-1))[0]}")


def assert_same_logits(a: np.ndarray, b: np.ndarray, dtype: str, what: str = "") -> None:
    """Two engine runs of the same positions, cut differently. In fp32 the kernels
    add in an order that does not depend on the cut, so the logits are equal to
    the bit; in bf16 the library GEMM may choose another algorithm for another
    shape, and they agree within rounding."""
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    if dtype == "float32":
        bad = np.flatnonzero((a != b).any(axis=-1))
        assert bad.size == 0, (f"{what}: rows {bad[:8].tolist()} differ, first by "
                               f"{np.abs(a[bad[0]] - b[bad[0]]).max():.3e}")
    else:
        bound = BF16_RTOL * b.astype(np.float64).std(axis=-1, keepdims=True)
        diff = np.abs(a.astype(np.float64) - b)
        bad = np.flatnonzero((diff > bound).any(axis=-1))
        assert bad.size == 0, (f"{what}: rows {bad[:8].tolist()} differ, first by "
                               f"{diff[bad[0]].max():.3e} (bound {bound[bad[0], 0]:.3e})")

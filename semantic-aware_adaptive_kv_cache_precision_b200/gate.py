"""Comparing two sets of logits of the same positions: the gate between the bfloat16 path
and the true 32-bit path of the same model.

The reference gates its engine against stored fp32 logits with two numbers
(`src/microinfer/gate.py:26-28, 31-40`): the share of positions whose argmax agrees (at
least 0.99) and the mean KL divergence (below 1e-3). Where it compares two ways of running
its own engine, an argmax that changed is excused only where the exact logits' two largest
values lie closer together than the bound on the difference
(`tests/test_chunked_prefill.py:44-45, 71-77`). Both rules are used here: a flip counts as
agreement only at a near tie.
"""

from __future__ import annotations

import numpy as np

TOP1_MIN = 0.99
KL_MAX = 1e-3
#: a logit of the bfloat16 path may differ from the exact one by this share of the standard
#: deviation of its row (about ten bf16 roundings a layer; the tests use the same bound)
NEAR_TIE_RTOL = 6e-2


def kl_divergence(exact: np.ndarray, candidate: np.ndarray) -> np.ndarray:
    """KL(exact || candidate) of each row, from logits, in float64."""
    def log_softmax(z):
        z = z.astype(np.float64)
        z = z - z.max(-1, keepdims=True)
        return z - np.log(np.exp(z).sum(-1, keepdims=True))

    p, q = log_softmax(exact), log_softmax(candidate)
    return (np.exp(p) * (p - q)).sum(-1)


def compare_logits(candidate: np.ndarray, exact: np.ndarray) -> dict:
    """`candidate` and `exact`: [positions, vocab]. Returns the gate's numbers:
    `top1_raw` (share of equal argmax), `top1_agreement` (flips at near ties counted as
    agreement), `near_tie_flips`, `hard_flips` (flips away from a near tie), `mean_kl`,
    `max_abs_logit_diff`, `max_diff_over_std`, and `passed`."""
    exact = np.asarray(exact, dtype=np.float64)
    candidate = np.asarray(candidate, dtype=np.float64)
    if exact.shape != candidate.shape or exact.ndim != 2:
        raise ValueError(f"logits of shapes {candidate.shape} and {exact.shape} cannot be compared")
    std = exact.std(-1)
    top_two = np.sort(exact, -1)[:, -2:]
    near_tie = (top_two[:, 1] - top_two[:, 0]) < NEAR_TIE_RTOL * std
    flipped = exact.argmax(-1) != candidate.argmax(-1)
    kl = kl_divergence(exact, candidate)
    diff = np.abs(exact - candidate)
    report = {
        "positions": int(exact.shape[0]),
        "top1_raw": float(1.0 - flipped.mean()),
        "top1_agreement": float(1.0 - (flipped & ~near_tie).mean()),
        "near_tie_flips": int((flipped & near_tie).sum()),
        "hard_flips": int((flipped & ~near_tie).sum()),
        "mean_kl": float(kl.mean()),
        "max_abs_logit_diff": float(diff.max()),
        "max_diff_over_std": float((diff.max(-1) / std).max()),
    }
    report["passed"] = bool(report["top1_agreement"] >= TOP1_MIN and report["mean_kl"] < KL_MAX)
    return report

"""The gate's arithmetic on made-up logits. No GPU."""

import numpy as np

from semantic_aware_adaptive_kv_cache_precision_b200.gate import compare_logits, kl_divergence


def test_kl_is_zero_for_equal_rows_and_positive_otherwise():
    rng = np.random.default_rng(0)
    z = rng.standard_normal((5, 40))
    np.testing.assert_allclose(kl_divergence(z, z + 3.0), 0, atol=1e-12)   # a shift is no change
    assert (kl_divergence(z, z + 0.1 * rng.standard_normal(z.shape)) > 0).all()


def test_a_flip_is_excused_only_at_a_near_tie():
    rng = np.random.default_rng(1)
    exact = rng.standard_normal((200, 50))
    exact[:, 7] = 6.0                                   # a clear winner everywhere
    candidate = exact + 1e-3 * rng.standard_normal(exact.shape)
    report = compare_logits(candidate, exact)
    assert report["passed"] and report["top1_raw"] == 1.0 and report["hard_flips"] == 0
    # row 0: a near tie that tips over; row 1: a clear winner that loses
    exact[0, 8] = 6.0 - 1e-4
    candidate = exact.copy()
    candidate[0, 8] += 1e-3
    report = compare_logits(candidate, exact)
    assert report["near_tie_flips"] == 1 and report["hard_flips"] == 0 and report["passed"]
    assert report["top1_raw"] < 1.0 == report["top1_agreement"]
    candidate[1, 9] = 7.0
    report = compare_logits(candidate, exact)
    assert report["hard_flips"] == 1 and report["top1_agreement"] == 1 - 1 / 200
    candidate[2:12, 9] = 7.0                            # eleven hard flips of 200: below 99 %
    assert not compare_logits(candidate, exact)["passed"]

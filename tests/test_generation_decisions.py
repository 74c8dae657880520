"""The generation loop's decisions. No GPU."""

import numpy as np
import pytest

from semantic_aware_adaptive_kv_cache_precision_b200.engine.generate import (
    RequestState, blocks_needed, check_prompt, check_window, plan_batches, plan_prefill,
    positions_needed)


def test_positions_needed_never_feeds_the_last_token():
    assert positions_needed(10, 5) == 14
    assert positions_needed(10, 1) == 10
    assert blocks_needed(64, 1) == 1 and blocks_needed(64, 2) == 2


def test_batches_respect_count_and_cache():
    assert plan_batches([5, 11, 17], 8, 64, 1024) == [[0, 1, 2]]
    assert plan_batches([5] * 5, 8, 2, 1024) == [[0, 1], [2, 3], [4]]
    # each request needs 2 blocks; the cache has 3
    assert plan_batches([100, 100, 100], 4, 64, 192) == [[0], [1], [2]]
    assert plan_batches([100, 10, 100], 4, 64, 192) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="request 1 needs"):
        plan_batches([5, 500], 8, 64, 256)
    with pytest.raises(ValueError):
        plan_batches([5], 8, 0, 256)


def test_prefill_is_one_step_unless_too_large():
    assert plan_prefill([5, 11, 17], 100) == [[(0, 0, 5), (1, 0, 11), (2, 0, 17)]]
    steps = plan_prefill([5, 11, 17], 8)
    assert steps == [[(0, 0, 5), (1, 0, 3)], [(1, 3, 8)], [(2, 0, 8)], [(2, 8, 8)], [(2, 16, 1)]]
    fed = {}
    for step in steps:
        assert sum(n for _, _, n in step) <= 8
        for i, a, n in step:
            assert fed.get(i, 0) == a
            fed[i] = a + n
    assert fed == {0: 5, 1: 11, 2: 17}


def test_request_ends_at_stop_token_or_length():
    r = RequestState(0, np.array([1, 2]))
    r.accept(5, {9}, 3)
    assert not r.finished
    r.accept(9, {9}, 3)
    assert r.finished and r.reason == "stop" and r.out == [5, 9]
    r = RequestState(1, np.array([1]))
    for t in (4, 4, 4):
        r.accept(t, set(), 3)
    assert r.reason == "length"
    r = RequestState(2, np.array([1]))
    r.accept(9, {9}, 1)
    assert r.reason == "stop"          # a stop token on the last allowed token is a stop


def test_prompt_checks():
    assert check_prompt([1, 2, 3], 10).dtype == np.int32
    with pytest.raises(ValueError, match="1-D"):
        check_prompt([[1, 2]], 10)
    with pytest.raises(ValueError, match="empty"):
        check_prompt([], 10)
    with pytest.raises(ValueError, match="integers"):
        check_prompt([1.5], 10)
    with pytest.raises(ValueError, match=r"\[0, 10\)"):
        check_prompt([3, 10], 10)
    with pytest.raises(ValueError, match="context window"):
        check_window(129, 128)
    check_window(128, 128)

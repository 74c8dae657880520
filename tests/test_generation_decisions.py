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


# ---- the decode loop that runs a step ahead of the tokens it has read -------------------------

def _fake_model(request, step):
    """The token request `request` draws as its `step`-th (a fixed function of both)."""
    return (request * 7 + step * 3) % 11


def _run_ahead(prompts, max_new, stops, full_at=None):
    """decode_ahead over a fake device that remembers what was launched."""
    from semantic_aware_adaptive_kv_cache_precision_b200.cache.allocator import CacheFull
    from semantic_aware_adaptive_kv_cache_precision_b200.engine.generate import (
        RequestState, decode_ahead)
    requests = [RequestState(i, np.zeros(n, np.int32)) for i, n in enumerate(prompts)]
    log = {"launches": [], "unread_at_launch": [], "finished": [], "exhausted": []}
    live = []
    for r in requests:
        r.drawn = 1
        r.accept(_fake_model(r.index, 0), stops, max_new)
        if r.finished:
            log["finished"].append(r.index)
        else:
            live.append(r)
    first = [r.out[0] for r in live]
    unread = {"n": 0}

    def launch(step_requests, feed, rows):
        if full_at is not None and len(log["launches"]) == full_at:
            raise CacheFull("no block left")
        # the tokens fed are those the step before chose for the same requests
        fed = [feed[j] for j in rows]
        for r, t in zip(step_requests, fed):
            assert t == _fake_model(r.index, r.drawn - 1), "a request was fed another's token"
        log["launches"].append([r.index for r in step_requests])
        log["unread_at_launch"].append(unread["n"])
        unread["n"] += 1
        return [_fake_model(r.index, r.drawn) for r in step_requests]

    def read(handle):
        unread["n"] -= 1
        return list(handle)

    decode_ahead(live, first, max_new, stops, launch, read,
                 on_finish=lambda r: log["finished"].append(r.index),
                 on_exhausted=lambda r, why: log["exhausted"].append((r.index, why)))
    return requests, log


def _plain_loop(prompts, max_new, stops):
    out = []
    for i in range(len(prompts)):
        tokens = []
        while True:
            tokens.append(_fake_model(i, len(tokens)))
            if tokens[-1] in stops or len(tokens) >= max_new:
                break
        out.append(tokens)
    return out


@pytest.mark.parametrize("max_new", [1, 2, 3, 9])
@pytest.mark.parametrize("stops", [frozenset(), frozenset({4}), frozenset({0, 6})])
def test_running_a_step_ahead_gives_the_same_tokens(max_new, stops):
    prompts = [3, 5, 2, 8, 1]
    requests, log = _run_ahead(prompts, max_new, stops)
    assert [r.out for r in requests] == _plain_loop(prompts, max_new, stops)
    assert sorted(log["finished"]) == list(range(len(prompts))) and not log["exhausted"]
    # every launch but the first is made with exactly one step unread: the loop is one ahead
    assert log["unread_at_launch"] == ([0] + [1] * (len(log["launches"]) - 1))[:len(log["launches"])]
    for r in requests:
        steps_run = sum(r.index in step for step in log["launches"])
        needed = len(r.out) - 1
        # a request whose count was complete is never run again; one that met a stop token
        # runs at most one step too many
        assert steps_run == needed or (r.reason == "stop" and steps_run == needed + 1)
        if r.reason == "length":
            assert steps_run == needed


def test_a_full_cache_ends_what_is_left_after_reading_what_was_in_flight():
    requests, log = _run_ahead([3, 4, 5], max_new=8, stops=frozenset(), full_at=2)
    # two steps ran, their tokens were read (three tokens each with the prefill's), then the
    # third launch found the cache full
    assert [len(r.out) for r in requests] == [3, 3, 3]
    assert [i for i, _ in log["exhausted"]] == [0, 1, 2]
    assert all("no block" in why for _, why in log["exhausted"])


def test_stop_ids_come_from_generation_config_if_there_is_one(tmp_path):
    import json
    from semantic_aware_adaptive_kv_cache_precision_b200.engine.generate import stop_ids_of_folder
    assert stop_ids_of_folder(None, (7,)) == frozenset({7})
    assert stop_ids_of_folder(tmp_path, (7, 8)) == frozenset({7, 8})     # no such file
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5}))
    assert stop_ids_of_folder(tmp_path, (7,)) == frozenset({5})
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [5, 9]}))
    assert stop_ids_of_folder(tmp_path, (7,)) == frozenset({5, 9})
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 0.7}))
    assert stop_ids_of_folder(tmp_path, (7,)) == frozenset({7})

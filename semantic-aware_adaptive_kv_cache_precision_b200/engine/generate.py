"""The decisions of the generation loop, apart from any device work.

Which requests form a batch, how a long prefill is cut into steps, when a
request is finished and why. Everything here is plain Python over lists, so it
is tested without a GPU. The loop itself (`Engine.generate`) asks these
functions and runs the steps. The rules follow the reference's loop
(`src/microinfer/engine.py:1180-1206, 1229-1260`): a stop token ends a request
and is kept in its output; the last new token is never fed back, so a request
needs `len(prompt) + max_new_tokens - 1` positions.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ..cache import BLOCK
from ..cache.allocator import CacheFull

PREFILLING, DECODING = "prefilling", "decoding"
COMPLETE, EXHAUSTED = "complete", "exhausted"


@dataclass(frozen=True)
class Ending:
    """How a request ended (`src/microinfer/engine.py:184-192`): `state` COMPLETE
    or EXHAUSTED, the positions its cache held, its new tokens, and why
    ('stop': a stop token; 'length': max_new_tokens; or the cache's message)."""
    state: str
    positions: int
    tokens: np.ndarray
    reason: str = ""


def positions_needed(prompt_len: int, max_new_tokens: int) -> int:
    return prompt_len + max(max_new_tokens, 1) - 1


def blocks_needed(prompt_len: int, max_new_tokens: int) -> int:
    return -(-positions_needed(prompt_len, max_new_tokens) // BLOCK)


def plan_batches(prompt_lens: list, max_new_tokens: int, max_batch: int,
                 max_tokens: int) -> list[list[int]]:
    """Cut the requests, in their order, into batches that start together: at most
    `max_batch` requests, and no more cache blocks than `max_tokens` positions
    give, counting every request at its longest."""
    if max_batch <= 0:
        raise ValueError(f"max_batch must be positive, got {max_batch}")
    budget = max_tokens // BLOCK
    batches, current, used = [], [], 0
    for i, n in enumerate(prompt_lens):
        need = blocks_needed(n, max_new_tokens)
        if need > budget:
            raise ValueError(f"request {i} needs {need * BLOCK} cache positions "
                             f"({n} prompt + {max_new_tokens} new), the cache holds "
                             f"{budget * BLOCK}")
        if current and (len(current) >= max_batch or used + need > budget):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
    return batches


def plan_prefill(prompt_lens: list, max_step_tokens: int) -> list[list[tuple]]:
    """Cut the prefill of a batch into steps of at most `max_step_tokens` tokens.
    Each step is a list of (sequence index, first token, count). Normally one
    step takes every prompt whole; a batch whose prompts together exceed the
    limit is fed in order, a long prompt continuing in the next step."""
    if max_step_tokens <= 0:
        raise ValueError(f"max_step_tokens must be positive, got {max_step_tokens}")
    steps, current, room = [], [], max_step_tokens
    for i, n in enumerate(prompt_lens):
        done = 0
        while done < n:
            take = min(n - done, room)
            current.append((i, done, take))
            done += take
            room -= take
            if room == 0:
                steps.append(current)
                current, room = [], max_step_tokens
    if current:
        steps.append(current)
    return steps


@dataclass
class RequestState:
    index: int                       # the request's number among all requests of the call
    prompt: np.ndarray
    out: list = field(default_factory=list)
    reason: str = ""                 # '' while running
    drawn: int = 0                   # tokens chosen for it so far, read back by the host or not

    @property
    def finished(self) -> bool:
        return bool(self.reason)

    def accept(self, token: int, stop_ids, max_new_tokens: int) -> None:
        """Take a newly chosen token and decide whether the request goes on."""
        self.out.append(int(token))
        if int(token) in stop_ids:
            self.reason = "stop"
        elif len(self.out) >= max_new_tokens:
            self.reason = "length"


def decode_ahead(live: list, first_feed, max_new_tokens: int, stop_ids, launch, read,
                 on_token=None, on_finish=None, on_exhausted=None) -> None:
    """The decode loop of one batch, one step ahead of the tokens the host has read.

    `live`: requests whose first token (from the prefill) has been accepted and that go
    on; `first_feed`: whatever `launch` needs to find those first tokens (row i belongs to
    live[i]). `launch(requests, feed, rows)` starts a step in which requests[j] is fed row
    rows[j] of the tokens of `feed` (the first feed, or what the launch before returned)
    and a token is chosen for each; it returns at once with a handle, or raises
    `CacheFull`. `read(handle)` waits for those tokens and returns them as ints.

    Step t + 1 is launched BEFORE the tokens of step t are read: its inputs are taken
    where step t left them, so the host's work overlaps the device's. Who runs in step
    t + 1 is decided without them: everyone of step t but the requests whose count is
    complete. A request that turns out to have ended at a stop token in step t has then
    run one step too many; that step's token for it is thrown away. `on_token(request,
    token)` and `on_finish(request)` are called as tokens are read, in order;
    `on_exhausted(request, message)` for those a full cache cuts short.
    """
    def settle(step):
        requests, handle = step
        for r, token in zip(requests, read(handle)):
            if r.finished:
                continue                      # it ended a step earlier: this one was run in vain
            r.accept(token, stop_ids, max_new_tokens)
            if on_token:
                on_token(r, token)
            if r.finished and on_finish:
                on_finish(r)

    in_flight = None
    feed, rows = first_feed, list(range(len(live)))
    while live:
        try:
            handle = launch(live, feed, rows)
        except CacheFull as exc:
            if in_flight is not None:
                settle(in_flight)
                in_flight = None
            for r in live:
                if not r.finished and on_exhausted:
                    on_exhausted(r, str(exc))
            return
        for r in live:
            r.drawn += 1
        if in_flight is not None:
            settle(in_flight)
        in_flight = (live, handle)
        after = [j for j, r in enumerate(live) if r.drawn < max_new_tokens and not r.finished]
        feed, rows, live = handle, after, [live[j] for j in after]
    if in_flight is not None:
        settle(in_flight)


def stop_ids_of_folder(model_dir, configured=()) -> frozenset:
    """The end-of-sequence ids generation stops at: `eos_token_id` of the folder's
    generation_config.json, a number or a list (`src/microinfer/engine.py:1148-1153`; the
    instruct checkpoints list two there), else the ids that config.json gave
    (`configured`)."""
    import json
    from pathlib import Path
    if model_dir is not None:
        path = Path(model_dir) / "generation_config.json"
        if path.is_file():
            eos = json.loads(path.read_text()).get("eos_token_id")
            if eos is not None:
                return frozenset(int(e) for e in (eos if isinstance(eos, list) else [eos]))
    return frozenset(int(e) for e in configured)


def check_prompt(ids, vocab_size: int, what: str = "token_ids") -> np.ndarray:
    """One sequence of token ids, as the reference checks it
    (`src/microinfer/engine.py:1836-1851`)."""
    arr = np.asarray(ids)
    if arr.ndim != 1:
        raise ValueError(f"{what} must be one sequence, 1-D; got shape {arr.shape}")
    if arr.size == 0:
        raise ValueError(f"{what} is empty")
    if not np.issubdtype(arr.dtype, np.integer):
        raise ValueError(f"{what} must be integers, got {arr.dtype}")
    if arr.min() < 0 or arr.max() >= vocab_size:
        raise ValueError(f"token ids must lie in [0, {vocab_size}); "
                         f"got [{arr.min()}, {arr.max()}]")
    return arr.astype(np.int32)


def check_window(positions: int, window: int) -> None:
    """`src/microinfer/engine.py:1853-1860`."""
    if positions > window:
        raise ValueError(f"{positions} positions exceed the model's context window of "
                         f"{window}: shorten the prompt or ask for fewer new tokens")

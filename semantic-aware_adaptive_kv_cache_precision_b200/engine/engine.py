"""The engine: a model, its cache, the step function and the generation loop.

The Python entry point follows the reference's `Engine`
(`src/microinfer/engine.py:822-833, 927-974, 1157-1206`): `Engine(model_dir)`,
`load_weights()`, `generate(prompt, max_new_tokens=64, *, stop_at_eos=True,
report=None)`, `forward(token_ids)`, `eos_token_ids`, `ending`. Where the
reference runs one sequence, this engine runs batches: `generate` also takes a
list of prompts, and `step` feeds any batch of sequences that start together.
"""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from .. import ops, sampling
from ..ops import _lib
from ..cache import BLOCK, CacheFull, SequenceCache
from ..config import config_from_dict, config_from_folder
from .generate import (decode_ahead, COMPLETE, DECODING, EXHAUSTED, PREFILLING, Ending, RequestState,
                       check_prompt, check_window, plan_batches, plan_prefill, positions_needed,
                       stop_ids_of_folder)
from .model import DecoderModel
from .step import StepStager

DEFAULT_MAX_TOKENS = 16384
DEFAULT_MAX_BATCH = 64
DEFAULT_MAX_STEP_TOKENS = 16384


class Engine:
    """`model_dir`: a folder with config.json and model.safetensors. Instead of a
    folder, `config=` (a config.json dict or a configuration object) with
    `random_seed=` builds the model with random weights on the device.

    `dtype`: 'bfloat16' (the serving kernels) or 'float32' (everything in true
    32-bit). `max_tokens`: cache positions over all live sequences, each
    sequence counted in blocks of 64. `max_batch`: most sequences in one batch.
    """

    def __init__(self, model_dir=None, *, config=None, dtype: str = "bfloat16",
                 max_tokens: int = DEFAULT_MAX_TOKENS, max_batch: int = DEFAULT_MAX_BATCH,
                 max_step_tokens: int = DEFAULT_MAX_STEP_TOKENS, random_seed: int | None = None,
                 device="cuda", poison_freed: bool = False, cuda_graphs: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this library runs its own sm_100a kernels "
                               "and has no CPU implementation")
        if (model_dir is None) == (config is None):
            raise ValueError("give either a model folder or config=")
        self.model_dir = None if model_dir is None else Path(model_dir)
        if config is None:
            self.config = config_from_folder(self.model_dir)
        else:
            self.config = config_from_dict(config) if isinstance(config, dict) else config
        self.dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(dtype, dtype)
        self.device = torch.device(device)
        self.random_seed = random_seed
        self.max_tokens, self.max_batch = int(max_tokens), int(max_batch)
        self.max_step_tokens = int(max_step_tokens)
        self.poison_freed = poison_freed
        self.spec = self.config.model_spec()
        self.model = DecoderModel(self.spec, self.dtype, self.device)
        self.cache: SequenceCache | None = None
        self._stager = StepStager(self.device)
        #: decode steps (one token per sequence, logits wanted for each) are captured in a
        #: CUDA graph per batch shape and replayed: the step's integers live at fixed
        #: device addresses, so a replay needs only the one copy that refreshes them
        self.cuda_graphs = cuda_graphs
        self._graphs: dict = {}
        self._graph_pool = None
        self._decode_ran_eagerly = False
        self.graph_failure = None
        self._prefill_graphs = {}
        #: steps of up to this many tokens are captured when their shape repeats (0: never);
        #: at most `prefill_graph_count` of them are kept
        self.prefill_graph_tokens = 8192
        self.prefill_graph_count = 8
        self.ending = None
        self.endings: list = []
        self._loaded = False
        self._tokenizer = None

    # -- loading ----------------------------------------------------------------

    def load_weights(self) -> "Engine":
        """Check the checkpoint against the configuration, then put every tensor on
        the device; a model is never half loaded. If the device has no room the call
        raises `OutOfDeviceMemory` and the engine stays as it was before the call."""
        with torch.cuda.device(self.device):
            if self.model_dir is not None:
                self.model.load(self.model_dir)
            else:
                self.model.load_random(0 if self.random_seed is None else self.random_seed)
        self._loaded = True
        return self

    def release(self) -> None:
        """Give up the cache, the graphs that were captured over it and over the weights, and
        the TMA descriptors that were kept for both (a later tensor at one of their addresses
        then gets a descriptor of its own). The weights stay; the next step builds a new
        cache. Called when the engine is dropped."""
        from .. import ops
        self._graphs.clear()
        self._prefill_graphs.clear()
        held = [] if self.model.arena is None else [self.model.arena.buffer]
        if self.cache is not None:
            for group in self.cache.groups:
                held += [group.keys, group.values]
        try:
            ops.forget_descriptors(*held)
        except Exception:            # the interpreter may be shutting down
            pass
        self.cache = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    def _need_loaded(self) -> None:
        if not self._loaded:
            raise RuntimeError("no weights on the device; call load_weights() first")

    def _need_cache(self) -> SequenceCache:
        if self.cache is None:
            self._need_loaded()
            act = torch.float32 if self.dtype == "float32" else torch.bfloat16
            # built whole before the engine keeps it: if the device has no room
            # (`OutOfDeviceMemory`) the engine still has no cache and can be asked again
            cache = SequenceCache(self.model.cache_needs(), self.max_tokens,
                                  self.spec.max_positions, act, self.device,
                                  max_slots=min(-(-self.max_tokens // BLOCK), 4096),
                                  poison_freed=self.poison_freed)
            self.model.prepare(cache.max_seq_len)
            self.cache = cache
        return self.cache

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    @property
    def eos_token_ids(self) -> frozenset:
        """generation_config.json's eos_token_id if the folder has one
        (`src/microinfer/engine.py:1148-1153`), else config.json's."""
        return stop_ids_of_folder(self.model_dir, self.spec.stop_token_ids)

    @property
    def tokenizer(self):
        """The model folder's own tokenizer.json through the `tokenizers` package
        (`src/microinfer/engine.py:1133-1140`). Token ids in and out are the contract of
        this library; text is a convenience for folders that carry a tokenizer."""
        if self._tokenizer is None:
            path = None if self.model_dir is None else self.model_dir / "tokenizer.json"
            if path is None or not path.is_file():
                raise RuntimeError("this model has no tokenizer.json: give token ids, not text")
            try:
                from tokenizers import Tokenizer
            except ImportError:
                raise RuntimeError("the `tokenizers` package is not installed: give token "
                                   "ids, not text") from None
            self._tokenizer = Tokenizer.from_file(str(path))
        return self._tokenizer

    def encode(self, text: str) -> np.ndarray:
        """Token ids (int32) of `text` (`src/microinfer/engine.py:1142-1143`)."""
        return np.asarray(self.tokenizer.encode(text).ids, dtype=np.int32)

    def decode(self, token_ids) -> str:
        """Text of token ids (`src/microinfer/engine.py:1145-1146`)."""
        return self.tokenizer.decode([int(t) for t in token_ids])

    def footprint(self) -> dict:
        """Bytes on the device: weights, cache, and what the device reports."""
        free, total = torch.cuda.mem_get_info(self.device)
        return {"weights": self.model.weight_bytes,
                "kv_cache": 0 if self.cache is None else self.cache.nbytes,
                "device_free": free, "device_total": total}

    # -- the step function ----------------------------------------------------------

    def open(self, count: int = 1) -> list[int]:
        """Take cache slots for `count` new sequences."""
        return self._need_cache().open(count)

    def close(self, slots) -> None:
        """End sequences; what they hold goes back to the cache."""
        self._need_cache().close(slots)

    def next_tokens(self, slots: list, device_tokens: torch.Tensor) -> torch.Tensor:
        """One greedy decode step: feed `device_tokens[i]` (int32 [len(slots)], on the device)
        to the sequence in `slots[i]` and return the token each sequence chooses next, int32
        [len(slots)] on the device, VALID UNTIL THE NEXT STEP of this engine (copy it, or
        start its copy to the host, before that). It is `sampling.choose(step(slots,
        device_tokens=...))` with the choice inside the step's captured graph: the tokens are
        written where the next step reads its tokens, so feeding a call with what the call
        before returned copies nothing, and the logits are not copied out of the graph."""
        return self.step(slots, device_tokens=device_tokens, _greedy=True)

    def step(self, slots: list, new_tokens: list | None = None, want: list | None = None, *,
             device_tokens: torch.Tensor | None = None,
             hidden_states: list | None = None, _greedy: bool = False) -> torch.Tensor:
        """Feed `new_tokens[i]` to the sequence in `slots[i]`, after what its cache
        already holds, all sequences as one batch. Returns fp32 logits
        [wanted, vocab] on the device for `want[i]`, the places among
        `new_tokens[i]` whose logits are asked for, in the order of the sequences
        (default: each sequence's last token).

        `device_tokens` (int32 [len(slots)], on the device) instead of `new_tokens`: one
        token for each sequence, taken from the device on the stream, so that a step can be
        launched before the host has read the tokens the step before it chose.

        The sequences of a step need not be at the same place: some may start (a prompt),
        some go on with a further piece of their prompt, some with one token, all in the one
        batch.

        `hidden_states` (a list): fp32 copies [tokens, hidden] of the residual stream are
        appended to it, after the embedding, after every layer call but the last, and after
        the final norm (the reference's order, `src/microinfer/model.py:355-364, 398-402`);
        such a step runs kernel by kernel."""
        cache = self._need_cache()
        if device_tokens is not None:
            if new_tokens is not None:
                raise ValueError("give new_tokens or device_tokens, not both")
            if device_tokens.dtype != torch.int32 or device_tokens.shape != (len(slots),) \
                    or not device_tokens.is_cuda:
                raise ValueError("device_tokens: int32 [len(slots)] on the engine's device")
            new_tokens = [(0,)] * len(slots)
        if len(slots) != len(new_tokens) or not slots:
            raise ValueError("step needs as many token lists as slots, and at least one")
        if len(set(slots)) != len(slots):
            raise ValueError("a sequence appears twice in one step")
        counts = [len(t) for t in new_tokens]
        if min(counts) <= 0:
            raise ValueError("every sequence of a step must bring at least one token")
        starts = [int(cache.lengths[s]) for s in slots]
        ends = [s + c for s, c in zip(starts, counts)]
        if want is None:
            want = [[c - 1] for c in counts]
        rows, base = [], 0
        for w, c in zip(want, counts):
            for p in w:
                if not 0 <= p < c:
                    raise ValueError(f"wanted place {p} is outside the {c} tokens brought")
                rows.append(base + p)
            base += c
        with torch.cuda.device(self.device):
            cache.reserve(slots, ends)
            ctx = self._stager.build(slots, new_tokens, starts, rows, cache.tables_for(slots),
                                     device_tokens)
            if hidden_states is not None:
                x = self.model.hidden(ctx, cache, capture=hidden_states)
                hidden_states.append(self.model.final_states(x))
                logits = self.model.logits(x, ctx.want) if rows else torch.empty(
                    (0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
            elif self.cuda_graphs and self.model.graph_safe and ctx.is_decode \
                    and rows == list(range(len(slots))):
                logits = self._decode_by_graph(ctx, cache, _greedy)
                if _greedy:                      # (tokens, chosen inside the graph)
                    cache.advance(slots, ends)
                    return logits
            elif self.cuda_graphs and self.model.graph_safe and 0 < len(rows) <= 64 \
                    and ctx.tokens <= self.prefill_graph_tokens:
                logits = self._prefill_by_graph(ctx, cache, (tuple(counts), tuple(starts),
                                                             tuple(rows)))
            else:
                x = self.model.hidden(ctx, cache)
                logits = self.model.logits(x, ctx.want) if rows else torch.empty(
                    (0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
            cache.advance(slots, ends)
            return ops.choose(logits) if _greedy else logits

    @staticmethod
    def _slots_in_key(ctx, cache) -> tuple:
        """What a captured step keeps of the host's view of it. A graph replays the launches
        it was captured with, Python integers included. Per-sequence state is indexed by slot
        (`view.state[slot]` with the host's `step.host_slots`), so a graph of a model that
        has state belongs to the slots it was captured on; keys and values are reached
        through block lists on the device, so a model without state shares its graphs among
        all slots. (`step.starts`, `max_position` and `max_len` change from one replay to
        the next: a part whose launches depend on them is not `graph_safe`.)"""
        return tuple(ctx.host_slots) if cache.states else ()

    def _decode_by_graph(self, ctx, cache, greedy: bool = False) -> torch.Tensor:
        """Run a decode step through the CUDA graph of its shape (batch size and width of
        the block lists), capturing it the first time the shape comes up after one
        decode step has run eagerly (which loads and configures every kernel). With `greedy`
        the graph also chooses each sequence's next token and writes it into the step's own
        token field (`ctx.token_ids`, the same device address in every step of the shape),
        which is returned instead of the logits."""
        def run():
            logits = self.model.logits(self.model.hidden(ctx, cache), ctx.want)
            return ops.choose(logits, out=ctx.token_ids) if greedy else logits

        if not self._decode_ran_eagerly:
            self._decode_ran_eagerly = True
            return run()
        key = (ctx.sequences, tuple(tuple(t.shape) for t in ctx.tables), self._stager.generation,
               self._slots_in_key(ctx, cache), greedy)
        entry = self._graphs.get(key)
        if entry is None:
            if len(self._graphs) >= 64:                 # shapes come and go; keep the table small
                self._graphs.clear()
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            torch.cuda.synchronize(self.device)
            before = _lib.launches
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    out = run()
            except Exception as exc:
                self.graph_failure = repr(exc)      # kept for whoever wants to know why
                # A part of this model does something a graph cannot hold (it reads a value
                # back on the host, say, to route tokens). Nothing ran during the failed
                # capture; from now on this engine runs its decode steps kernel by kernel.
                self.cuda_graphs = False
                self._graphs.clear()
                _lib.launches = before
                try:
                    torch.cuda.synchronize(self.device)
                except Exception:
                    pass
                return run()
            entry = (graph, out, _lib.launches - before)
            self._graphs[key] = entry
            _lib.launches = before
        entry[0].replay()
        _lib.launches += entry[2]            # the kernels of this library inside the graph
        return ctx.token_ids if greedy else entry[1].clone()

    def _prefill_by_graph(self, ctx, cache, shape) -> torch.Tensor:
        """A step that is not a decode step, through a CUDA graph once its shape (how many
        tokens each sequence brings, after how many, and which logits are wanted) has come
        up before: the first time it runs kernel by kernel, the second time it is captured,
        from then on replayed. Launching a prefill's 400 kernels from Python takes 4 to 5 ms,
        longer than a short prompt's kernels run; a replay takes what the kernels take.
        Requests of a shape never seen again cost nothing but a dictionary entry."""
        key = (shape, tuple(tuple(t.shape) for t in ctx.tables), self._stager.generation,
               self._slots_in_key(ctx, cache))
        entry = self._prefill_graphs.get(key)
        if entry is None:                                   # first time: eagerly
            if len(self._prefill_graphs) >= 256:
                self._prefill_graphs.clear()
            out = self.model.logits(self.model.hidden(ctx, cache), ctx.want)
            self._prefill_graphs[key] = ctx.plans          # what the parts worked out for it
            return out
        if isinstance(entry, dict):                         # second time: capture
            captured = sum(1 for e in self._prefill_graphs.values() if isinstance(e, tuple))
            if captured >= self.prefill_graph_count:
                ctx.plans = entry
                return self.model.logits(self.model.hidden(ctx, cache), ctx.want)
            ctx.plans = entry                               # nothing is uploaded while capturing
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            torch.cuda.synchronize(self.device)
            before = _lib.launches
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    out = self.model.logits(self.model.hidden(ctx, cache), ctx.want)
            except Exception as exc:
                self.graph_failure = repr(exc)
                self.prefill_graph_tokens = 0               # no more attempts
                _lib.launches = before
                try:
                    torch.cuda.synchronize(self.device)
                except Exception:
                    pass
                return self.model.logits(self.model.hidden(ctx, cache), ctx.want)
            entry = (graph, out, _lib.launches - before, entry)
            self._prefill_graphs[key] = entry
            _lib.launches = before
        entry[0].replay()
        _lib.launches += entry[2]
        return entry[1].clone()

    # -- whole sequences ---------------------------------------------------------------

    def forward(self, token_ids, *, capture_hidden_states: bool = False):
        """fp32 logits (seq, vocab) for every position of one sequence
        (`src/microinfer/engine.py:1157-1178`). With `capture_hidden_states`, returns
        `(logits, hidden_states)`, the states fp32 (layer calls + 1, seq, hidden): the
        embedding's output, the stream after every layer call but the last, and the last
        one's after the final norm."""
        self._need_loaded()
        ids = check_prompt(token_ids, self.spec.vocab_size)
        check_window(len(ids), self.spec.max_positions)
        (slot,) = self.open(1)
        try:
            out, states = [], []
            for begin in range(0, len(ids), self.max_step_tokens):
                chunk = ids[begin:begin + self.max_step_tokens]
                captured = [] if capture_hidden_states else None
                out.append(self.step([slot], [chunk], [list(range(len(chunk)))],
                                     hidden_states=captured).cpu().numpy())
                if capture_hidden_states:
                    states.append(torch.stack([c.float() for c in captured]).cpu().numpy())
            logits = np.concatenate(out)
            if capture_hidden_states:
                return logits, np.concatenate(states, axis=1)
            return logits
        finally:
            self.close([slot])

    def cached_kv(self, token_ids) -> tuple[np.ndarray, np.ndarray]:
        """What the cache holds after prefilling one sequence: keys and values, each fp32
        (cache entries, seq, kv_heads, head_dim), read back from the blocks the sequence was
        given (`src/microinfer/engine.py:1819-1834`). Keys are as stored: rotated, WITH their
        projection's bias (the reference caches them without). A position that a windowed
        entry has already given back reads as NaN; an entry that keeps no keys and values
        (per-sequence state) is left out. All kept entries must have one shape."""
        self._need_loaded()
        ids = check_prompt(token_ids, self.spec.vocab_size)
        check_window(len(ids), self.spec.max_positions)
        cache = self._need_cache()
        (slot,) = self.open(1)
        try:
            for begin in range(0, len(ids), self.max_step_tokens):
                chunk = ids[begin:begin + self.max_step_tokens]
                self.step([slot], [chunk], [[]])
            torch.cuda.synchronize(self.device)
            keys, values = [], []
            for entry, need in enumerate(cache.needs):
                if entry not in cache.entry_group:
                    continue
                g, i = cache.entry_group[entry]
                group = cache.groups[g]
                if group.values is None:
                    continue
                blocks = group.tables[slot, :-(-len(ids) // BLOCK)]
                held = torch.as_tensor(np.maximum(blocks, 0), dtype=torch.long, device=self.device)

                def read(store):
                    rows = store[i][held].float()                  # [blocks, kv_heads, 64, d]
                    rows[torch.as_tensor(blocks < 0, device=self.device)] = float("nan")
                    rows = rows.permute(0, 2, 1, 3).reshape(-1, rows.shape[1], rows.shape[3])
                    return rows[:len(ids)].cpu().numpy()

                keys.append(read(group.keys))
                values.append(read(group.values))
            return np.stack(keys), np.stack(values)
        finally:
            self.close([slot])

    # -- generation -------------------------------------------------------------------------

    def generate(self, prompt, max_new_tokens: int = 64, *, stop_at_eos: bool = True,
                 report=None, temperature: float = 0.0, seed: int = 0, stop_token_ids=None):
        """New token ids for one prompt (a 1-D sequence of ids, or text if the model folder
        has a tokenizer.json: returns one int32 array) or for a list of prompts (returns a
        list of int32 arrays).

        Prompts are taken in batches that start together; each batch prefills all
        its prompts in one step and then decodes one token per live request a
        step. A request ends after `max_new_tokens` or at a stop token, which is
        kept (`stop_at_eos`: the model's end-of-sequence ids; `stop_token_ids`
        replaces them), and leaves its batch at once. `temperature` 0 is greedy.
        `report(phase, positions, token)` is called after each prefill with token
        None and after each decoded token; for a list of prompts it gets the
        request's number as a fourth argument. `self.ending` (one prompt) or
        `self.endings` say how each request ended.
        """
        self._need_loaded()
        if isinstance(prompt, str):                    # text, if the folder has a tokenizer
            prompt = self.encode(prompt)
        single = not _is_list_of_sequences(prompt)
        prompts = [prompt] if single else list(prompt)
        prompts = [self.encode(p) if isinstance(p, str) else p for p in prompts]
        if max_new_tokens < 0:
            raise ValueError(f"max_new_tokens must not be negative, got {max_new_tokens}")
        ids = [check_prompt(p, self.spec.vocab_size, f"prompt {i}" if not single else "token_ids")
               for i, p in enumerate(prompts)]
        params = sampling.SamplingParams(float(temperature), int(seed))
        if max_new_tokens == 0:
            self.endings = [Ending(COMPLETE, 0, np.empty(0, np.int32), "length") for _ in ids]
            self.ending = self.endings[0] if single else None
            return self.endings[0].tokens if single else [e.tokens for e in self.endings]
        for p in ids:
            check_window(positions_needed(len(p), max_new_tokens), self.spec.max_positions)
        if stop_token_ids is not None:
            stops = frozenset(int(t) for t in stop_token_ids)
        else:
            stops = self.eos_token_ids if stop_at_eos else frozenset()
        if report is None:
            tell = lambda *a: None
        elif single:
            tell = lambda phase, positions, token, request: report(phase, positions, token)
        else:
            tell = report

        cache = self._need_cache()
        batches = plan_batches([len(p) for p in ids], max_new_tokens, self.max_batch,
                               cache.max_tokens)
        endings: dict[int, Ending] = {}
        for batch in batches:
            self._run_batch([RequestState(i, ids[i]) for i in batch], max_new_tokens, stops,
                            params, tell, endings)
        self.endings = [endings[i] for i in range(len(ids))]
        self.ending = self.endings[0] if single else None
        return self.endings[0].tokens if single else [e.tokens for e in self.endings]

    def _run_batch(self, requests, max_new_tokens, stops, params, tell, endings) -> None:
        cache = self._need_cache()
        slots = cache.open(len(requests))
        slot_of = {r.index: s for r, s in zip(requests, slots)}
        live = list(requests)

        def positions(r):           # what its cache holds: the last new token is never fed
            return len(r.prompt) + len(r.out) - 1

        def finish(r, state=COMPLETE, reason=None):
            endings[r.index] = Ending(state, positions(r), np.asarray(r.out, np.int32),
                                      reason or r.reason)
            cache.close([slot_of[r.index]])

        try:
            # prefill: every prompt whole, in one step unless the batch is too large
            try:
                plans = plan_prefill([len(r.prompt) for r in requests], self.max_step_tokens)
                logits = {}
                for plan in plans:
                    step_slots = [slots[i] for i, _, _ in plan]
                    tokens = [requests[i].prompt[a:a + n] for i, a, n in plan]
                    ends = [a + n == len(requests[i].prompt) for i, a, n in plan]
                    want = [[n - 1] if last else [] for (_, _, n), last in zip(plan, ends)]
                    out = self.step(step_slots, tokens, want)
                    row = 0
                    for (i, _, _), last in zip(plan, ends):
                        if last:
                            logits[i] = out[row]
                            row += 1
            except CacheFull as exc:
                for r in live:
                    endings[r.index] = Ending(EXHAUSTED, int(cache.lengths[slot_of[r.index]]),
                                              np.asarray(r.out, np.int32), str(exc))
                    cache.close([slot_of[r.index]])
                return
            first = self._choose(torch.stack([logits[i] for i in range(len(requests))]),
                                 params, live)
            for r, token in zip(live, self._read(first)):
                r.drawn = 1
                tell(PREFILLING, len(r.prompt), None, r.index)
                r.accept(token, stops, max_new_tokens)
            for r in [r for r in live if r.finished]:
                finish(r)
            keep = [j for j, r in enumerate(live) if not r.finished]
            live = [live[j] for j in keep]
            if len(keep) < len(requests):
                first = _Chosen(first.tokens[torch.as_tensor(keep, dtype=torch.long, device=self.device)], None, None)

            # decode: one token for each live request a step, a step ahead of the host
            def launch(step_requests, feed, rows):
                tokens = feed.tokens
                if len(rows) != tokens.shape[0]:
                    tokens = tokens[torch.as_tensor(rows, dtype=torch.long, device=self.device)]
                step_slots = [slot_of[r.index] for r in step_requests]
                if params.temperature == 0.0:          # the choice is part of the captured step
                    return self._on_its_way(self.next_tokens(step_slots, tokens))
                out = self.step(step_slots, device_tokens=tokens)
                return self._choose(out, params, step_requests)

            decode_ahead(live, first, max_new_tokens, stops, launch, self._read,
                         on_token=lambda r, t: tell(DECODING, positions(r), int(t), r.index),
                         on_finish=finish,
                         on_exhausted=lambda r, why: finish(r, EXHAUSTED, why))
        except BaseException:
            held = [slot_of[r.index] for r in requests if r.index not in endings]
            cache.close(held)
            raise

    def _choose(self, logits, params, live) -> "_Chosen":
        """A token for each row of `logits`, chosen on the device; its copy to the host is
        on its way (pinned memory) but nothing waits for it here."""
        return self._on_its_way(sampling.choose(logits, params, [r.index for r in live],
                                                [r.drawn for r in live]))

    @staticmethod
    def _on_its_way(tokens: torch.Tensor) -> "_Chosen":
        host = torch.empty(tokens.shape, dtype=torch.int32, pin_memory=True)
        host.copy_(tokens, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return _Chosen(tokens, host, done)

    def _read(self, chosen: "_Chosen") -> list[int]:
        chosen.done.synchronize()
        tokens = chosen.host.tolist()
        sampling.check_chosen(tokens, self.spec.vocab_size)
        return tokens


class _Chosen:
    """The tokens a step chose: on the device, and on their way to the host."""

    __slots__ = ("tokens", "host", "done")

    def __init__(self, tokens, host, done):
        self.tokens, self.host, self.done = tokens, host, done


def _is_list_of_sequences(prompt) -> bool:
    if isinstance(prompt, np.ndarray):
        return False              # an array is one prompt; a 2-D one is refused as such
    if isinstance(prompt, (list, tuple)) and prompt:
        return isinstance(prompt[0], (list, tuple, np.ndarray, str))
    return False

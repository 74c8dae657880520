"""The engine against the plain implementation, in 32-bit and in bfloat16: whole
prompts, the last 32 tokens one by one, batches of unequal lengths with slots
used again, long decoding, the first tokens of a sequence, and generation."""

import numpy as np
import pytest
import torch

import plain_model as plain
from conftest import TINY, prompts_for
from helpers import assert_close_to_plain, assert_same_logits, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "W", "C", "D"]


def engine_for(folder, dtype, **kw):
    from semantic_aware_adaptive_kv_cache_precision_b200 import Engine
    kw.setdefault("max_tokens", 2048)
    return Engine(folder, dtype=dtype, poison_freed=True, **kw).load_weights()


def stored(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@pytest.fixture(scope="module")
def engines(model_folders):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[name, dtype] = engine_for(model_folders(name, stored(dtype)), dtype)
        return made[name, dtype]

    return get


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(name, dtype, engines, model_folders):
    engine = engines(name, dtype)
    folder = model_folders(name, stored(dtype))
    lengths = {"A": [5, 11, 17, 100], "B": [1, 7, 30, 64, 200], "W": [3, 69, 70, 71, 150, 300],
               "C": [1, 64, 129, 131, 400], "D": [2, 65, 300, 1100]}[name]
    # (1,100 tokens: long enough for the feed-forward's fused tcgen05 product in bf16)
    for ids in prompts_for(name, lengths):
        got = engine.forward(ids)
        assert_close_to_plain(got, plain_logits(folder, ids), dtype, f"{name} len {len(ids)}")
    engine.cache.check()
    assert engine.cache.slots.held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(name, dtype, engines, model_folders):
    engine = engines(name, dtype)
    folder = model_folders(name, stored(dtype))
    for ids in prompts_for(name, {"A": [40, 120], "B": [33, 130], "W": [100, 260],
                                 "C": [33, 300], "D": [150]}[name], seed=1):
        whole = engine.forward(ids)
        (slot,) = engine.open(1)
        head = len(ids) - 32
        rows = [engine.step([slot], [ids[:head]], [list(range(head))]).cpu().numpy()]
        for t in range(head, len(ids)):
            rows.append(engine.step([slot], [ids[t:t + 1]]).cpu().numpy())
        engine.close([slot])
        stepped = np.concatenate(rows)
        assert_same_logits(stepped, whole, dtype, f"{name} len {len(ids)} stepped vs whole")
        assert_close_to_plain(stepped, plain_logits(folder, ids), dtype, f"{name} stepped")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(name, dtype, model_folders):
    """Three batches in a cache that holds barely one of them: every slot and block
    is used again, freed blocks are filled with NaN, and the shorter requests of
    a batch end while the others go on decoding."""
    folder = model_folders(name, stored(dtype))
    engine = engine_for(folder, dtype, max_tokens=8 * 64)
    batches = {"A": [[5, 11, 17], [64, 3, 30], [1, 90, 65]],
               "B": [[1, 7, 30, 64], [2, 100, 33, 5], [64, 65, 1, 128]],
               "W": [[3, 75, 140], [71, 70, 69], [1, 200, 64]],
               "C": [[1, 140, 64], [100, 120, 60], [2, 250, 63]],
               "D": [[5, 130, 64], [1, 200, 33], [100, 3, 66]]}[name]
    extra = [6, 2, 9, 4]                    # decode steps per request; unequal, so some end early
    for b, lengths in enumerate(batches):
        prompts = prompts_for(name, [n + e for n, e in zip(lengths, extra)], seed=10 + b)
        want_all = [plain_logits(folder, p) for p in prompts]
        slots = engine.open(len(prompts))
        out = engine.step(slots, [p[:n] for p, n in zip(prompts, lengths)],
                          [list(range(n)) for n in lengths]).cpu().numpy()
        got = [[] for _ in prompts]
        at = 0
        for i, n in enumerate(lengths):
            got[i].append(out[at:at + n])
            at += n
        live = list(range(len(prompts)))
        fed = list(lengths)
        while live:
            out = engine.step([slots[i] for i in live],
                              [prompts[i][fed[i]:fed[i] + 1] for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1])
                fed[i] += 1
            done = [i for i in live if fed[i] == len(prompts[i])]
            if done:
                engine.close([slots[i] for i in done])     # shorter requests end earlier
                live = [i for i in live if i not in done]
            engine.cache.check()
        for i, p in enumerate(prompts):
            assert_close_to_plain(np.concatenate(got[i]), want_all[i], dtype,
                                  f"{name} batch {b} request {i}")
        assert engine.cache.slots.held == 0
        assert all(g.pool.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_rows_equal_single_rows(dtype, engines):
    """What else is in the batch changes nothing (to the bit in fp32)."""
    engine = engines("B", dtype)
    prompts = prompts_for("B", [9, 70, 1, 33], seed=3)
    alone = [engine.forward(p) for p in prompts]
    slots = engine.open(4)
    out = engine.step(slots, prompts, [list(range(len(p))) for p in prompts]).cpu().numpy()
    engine.close(slots)
    at = 0
    for p, a in zip(prompts, alone):
        assert_same_logits(out[at:at + len(p)], a, dtype, f"len {len(p)} in a batch vs alone")
        at += len(p)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype, engines, model_folders):
    engine = engines("W", dtype)
    folder = model_folders("W", stored(dtype))
    ids = prompts_for("W", [400], seed=4)[0]
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [ids[:3]], [[0, 1, 2]]).cpu().numpy()]
    for t in range(3, len(ids)):
        rows.append(engine.step([slot], [ids[t:t + 1]]).cpu().numpy())
    engine.close([slot])
    assert_close_to_plain(np.concatenate(rows), plain_logits(folder, ids), dtype, "long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(name, dtype, engines, model_folders):
    engine = engines(name, dtype)
    folder = model_folders(name, stored(dtype))
    ids = prompts_for(name, [4], seed=6)[0]
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [ids[t:t + 1]]).cpu().numpy() for t in range(4)]
    engine.close([slot])
    assert_close_to_plain(np.concatenate(rows), plain_logits(folder, ids), dtype, "first tokens")


def test_greedy_generation_through_the_entry_point(engines, model_folders):
    engine = engines("A", "float32")
    config, tensors = plain.read_model_folder(model_folders("A", "float32"))
    prompts = prompts_for("A", [5, 11, 17])
    want = [plain.generate(config, tensors, p, 8) for p in prompts]
    got = engine.generate([p.tolist() for p in prompts], 8, stop_at_eos=False)
    assert [g.tolist() for g in got] == want
    assert all(g.dtype == np.int32 for g in got)
    one = engine.generate(prompts[1], 8, stop_at_eos=False)
    assert one.tolist() == want[1] and engine.ending.state == "complete"
    # a stop token ends a request early and is kept; the others go on
    stop = want[0][2]
    got = engine.generate([p.tolist() for p in prompts], 8, stop_token_ids=[stop])
    for g, w, e in zip(got, want, engine.endings):
        cut = w.index(stop) + 1 if stop in w else len(w)
        assert g.tolist() == w[:cut]
        assert e.reason == ("stop" if stop in w else "length")
    assert engine.generate(prompts[0], 0).size == 0
    assert engine.cache.slots.held == 0
    # the loop runs a step ahead of the tokens it has read: short counts, and a stop token at
    # every place of every request, end where the plain loop ends
    for n in (1, 2, 3):
        got = engine.generate([p.tolist() for p in prompts], n, stop_at_eos=False)
        assert [g.tolist() for g in got] == [w[:n] for w in want]
    for place in range(8):
        for who in range(len(prompts)):
            stop = want[who][place]
            got = engine.generate([p.tolist() for p in prompts], 8, stop_token_ids=[stop])
            for g, w, e in zip(got, want, engine.endings):
                cut = w.index(stop) + 1 if stop in w else len(w)
                assert g.tolist() == w[:cut] and e.positions == len(g) + e.positions - len(g)
                assert e.reason == ("stop" if stop in w else "length")
            assert engine.endings[who].positions == len(prompts[who]) + len(got[who]) - 1
    assert engine.cache.slots.held == 0


def test_temperature_generation_matches_the_plain_sampler(engines, model_folders):
    engine = engines("B", "float32")
    config, tensors = plain.read_model_folder(model_folders("B", "float32"))
    prompts = prompts_for("B", [1, 7, 30, 64])
    want = [plain.generate(config, tensors, p, 16, temperature=0.8, seed=1234, request=i)
            for i, p in enumerate(prompts)]
    got = engine.generate([p.tolist() for p in prompts], 16, stop_at_eos=False,
                          temperature=0.8, seed=1234)
    assert [g.tolist() for g in got] == want
    greedy = engine.generate([p.tolist() for p in prompts], 16, stop_at_eos=False)
    assert [g.tolist() for g in greedy] != want
    # what a request draws does not depend on its batch: two batches of two
    small = Engine_like(engine, max_batch=2)
    again = small.generate([p.tolist() for p in prompts], 16, stop_at_eos=False,
                           temperature=0.8, seed=1234)
    assert [g.tolist() for g in again] == want


def Engine_like(engine, **kw):
    from semantic_aware_adaptive_kv_cache_precision_b200 import Engine
    return Engine(engine.model_dir, dtype=engine.dtype, max_tokens=2048, **kw).load_weights()


def test_generation_refuses_bad_requests(engines):
    engine = engines("A", "float32")
    with pytest.raises(ValueError, match="1-D"):
        engine.generate(np.zeros((2, 3), dtype=np.int64), 4)
    with pytest.raises(ValueError, match="empty"):
        engine.generate([], 4)
    with pytest.raises(ValueError, match=r"\[0, 512\)"):
        engine.generate([1, 512], 4)
    with pytest.raises(ValueError, match="context window"):
        engine.generate([1] * 120, 20)
    with pytest.raises(ValueError, match="negative"):
        engine.generate([1], -1)
    assert engine.cache is None or engine.cache.slots.held == 0


def test_reports_and_endings(engines):
    engine = engines("A", "float32")
    seen = []
    out = engine.generate([3, 4, 5], 4, stop_at_eos=False, report=lambda *a: seen.append(a))
    assert seen[0] == ("prefilling", 3, None)
    assert [s[0] for s in seen[1:]] == ["decoding"] * 3
    assert [s[2] for s in seen[1:]] == out[1:].tolist()
    assert [s[1] for s in seen[1:]] == [4, 5, 6]
    assert engine.ending.positions == 6 and engine.ending.reason == "length"


def test_cache_full_ends_requests_gracefully(model_folders):
    engine = engine_for(model_folders("A", "float32"), "float32", max_tokens=64)
    with pytest.raises(ValueError, match="cache holds"):
        engine.generate([1] * 60, 20, stop_at_eos=False)
    out = engine.generate([[1] * 30, [2] * 30], 5, stop_at_eos=False)     # one block: two batches
    assert all(len(o) == 5 for o in out)
    assert engine.cache.slots.held == 0
    # a step that outgrows the cache takes nothing and leaves the sequence as it was
    from semantic_aware_adaptive_kv_cache_precision_b200 import CacheFull
    (slot,) = engine.open(1)
    engine.step([slot], [[1] * 64])
    with pytest.raises(CacheFull, match="nothing was taken"):
        engine.step([slot], [[3]])
    assert engine.cache.lengths[slot] == 64
    engine.close([slot])
    engine.cache.check()


@pytest.mark.parametrize("name", ["C", "D"])
def test_graph_replayed_decode_equals_eager_decode(name, model_folders):
    """Decode steps are captured in a CUDA graph per batch shape and replayed; the logits
    must be those of the same steps run kernel by kernel. The sequences cross a block
    boundary and a change of the block lists' width on the way, and one ends early."""
    folder = model_folders(name, "bfloat16")
    prompts = prompts_for(name, [60, 500, 129], seed=40)
    runs = {}
    for graphs in (True, False):
        engine = engine_for(folder, "bfloat16", cuda_graphs=graphs)
        slots = engine.open(3)
        engine.step(slots, [p[:-30] for p in prompts])
        rows = []
        live = [0, 1, 2]
        for t in range(30):
            if t == 12:
                engine.close([slots[2]])
                live = [0, 1]
            out = engine.step([slots[i] for i in live],
                              [prompts[i][len(prompts[i]) - 30 + t:len(prompts[i]) - 29 + t]
                               for i in live])
            rows.append(out.cpu().numpy())
        engine.close([slots[i] for i in live])
        runs[graphs] = np.concatenate(rows)
        if graphs:
            assert len(engine._graphs) >= 2          # two batch sizes were captured
    np.testing.assert_array_equal(runs[True], runs[False])


@pytest.mark.parametrize("stored", ["float32", "float16"])
def test_bfloat16_mode_on_checkpoints_stored_in_other_types(stored, model_folders, tmp_path):
    """With dtype bfloat16, a tensor stored in 32 bits stays in 32 bits on the device (its
    products then run in true fp32), and float16 is kept as bfloat16. Either way the logits
    agree with the plain model within the bf16 bound."""
    import json
    import torch
    from semantic_aware_adaptive_kv_cache_precision_b200.weights import (SafetensorsFile,
                                                                          write_safetensors)
    src = model_folders("C", "float32")
    folder = tmp_path / f"c_{stored}"
    folder.mkdir()
    config = json.loads((src / "config.json").read_text())
    config["torch_dtype"] = stored
    (folder / "config.json").write_text(json.dumps(config))
    f = SafetensorsFile(src / "model.safetensors")
    dtype = {"float32": torch.float32, "float16": torch.float16}[stored]
    write_safetensors(folder / "model.safetensors", {n: f.tensor(n).to(dtype) for n in f.infos})
    engine = engine_for(folder, "bfloat16")
    held = {t.dtype for t in (engine.model.embed, engine.model.blocks[0].mixer.w_qkv,
                              engine.model.blocks[0].mixer_norm.weight)}
    assert held == ({torch.float32} if stored == "float32" else {torch.bfloat16})
    for ids in prompts_for("C", [70, 200], seed=50):
        whole = engine.forward(ids)
        assert_close_to_plain(whole, plain_logits(folder, ids), "bfloat16", f"stored {stored}")
        (slot,) = engine.open(1)
        rows = [engine.step([slot], [ids[:-5]], [list(range(len(ids) - 5))]).cpu().numpy()]
        rows += [engine.step([slot], [ids[t:t + 1]]).cpu().numpy() for t in range(len(ids) - 5, len(ids))]
        engine.close([slot])
        assert_same_logits(np.concatenate(rows), whole, "bfloat16", f"stored {stored}, stepped")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prefill_shape_that_repeats_is_replayed_from_a_graph(model_folders, dtype):
    """The third step of a shape runs as a graph replay: same logits as the engine that never
    captures, for other token ids than the graph was captured with, and after slots were
    given back and taken again."""
    folder = model_folders("B", dtype)
    graphs = engine_for(folder, dtype, max_tokens=2048)
    plain_steps = engine_for(folder, dtype, max_tokens=2048)
    plain_steps.cuda_graphs = False
    rng = np.random.default_rng(3)
    lengths = [70, 5, 131]
    for round_ in range(4):
        prompts = [rng.integers(0, 1000, n) for n in lengths]
        outs = []
        for engine in (graphs, plain_steps):
            slots = engine.open(3)
            first = engine.step(slots, prompts)
            second = engine.step(slots, [p[:2] for p in prompts], [[0, 1]] * 3)
            outs.append((first.cpu().numpy(), second.cpu().numpy()))
            engine.close(slots[::-1] if round_ % 2 else slots)
        for got, want in zip(outs[0], outs[1]):
            if dtype == "float32":
                np.testing.assert_array_equal(got, want)
            else:
                np.testing.assert_allclose(got, want, rtol=0, atol=1e-2 * np.abs(want).max())
    captured = [e for e in graphs._prefill_graphs.values() if isinstance(e, tuple)]
    assert len(captured) == 2 and graphs.graph_failure is None


def test_many_requests_in_batches_end_as_they_do_alone(model_folders):
    """Twenty-three requests of unequal lengths through batches of five, with a stop token
    that ends some of them early: each gets the tokens it gets alone (fp32: the same to the
    token), every slot comes back, and the endings say why."""
    folder = model_folders("A", "float32")
    engine = engine_for(folder, "float32", max_tokens=1024, max_batch=5)
    alone = engine_for(folder, "float32", max_tokens=1024, max_batch=1)
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, 512, int(n)).tolist() for n in rng.integers(1, 40, 23)]
    free = [alone.generate(p, 12, stop_at_eos=False).tolist() for p in prompts]
    counts = np.bincount(np.concatenate(free), minlength=512)
    stop = int(counts.argmax())                    # a token many of them produce
    want = [w[:w.index(stop) + 1] if stop in w else w for w in free]
    assert any(len(w) < 12 for w in want) and any(len(w) == 12 for w in want)
    got = engine.generate(prompts, 12, stop_token_ids=[stop])
    assert [g.tolist() for g in got] == want
    assert [e.reason for e in engine.endings] == ["stop" if w[-1] == stop else "length" for w in want]
    assert [e.positions for e in engine.endings] == [len(p) + len(w) - 1 for p, w in zip(prompts, want)]
    assert engine.cache.slots.held == 0
    engine.cache.check()

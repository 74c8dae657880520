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
                assert g.tolist() == w[:cut]
                assert e.reason == ("stop" if stop in w else "length")
            for p, g, e in zip(prompts, got, engine.endings):
                assert e.positions == len(p) + len(g) - 1      # the last token is never fed
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


# ---- steps whose sequences are at different places --------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_a_step_may_mix_starting_continuing_and_decoding_sequences(name, dtype, engines):
    """One step in which sequence a starts with 70 tokens, b goes on with 5 after 64 and c
    with 1 after 200; then a step in which a decodes, b brings 3 more and d starts. Every
    position's logits are those of its sequence run alone and whole: to the bit in 32-bit,
    within rounding in bfloat16."""
    engine = engines(name, dtype)
    a, b, c, d = prompts_for(name, [71, 72, 201, 9], seed=70)
    whole = {k: engine.forward(p) for k, p in zip("abcd", (a, b, c, d))}
    sa, sb, sc = engine.open(3)
    engine.step([sb, sc], [b[:64], c[:200]], [[], []])
    out = engine.step([sa, sb, sc], [a[:70], b[64:69], c[200:201]],
                      [list(range(70)), list(range(5)), [0]]).cpu().numpy()
    assert_same_logits(out[:70], whole["a"][:70], dtype, "a starts beside others")
    assert_same_logits(out[70:75], whole["b"][64:69], dtype, "b goes on by five")
    assert_same_logits(out[75:76], whole["c"][200:201], dtype, "c decodes one")
    engine.close([sc])
    (sd,) = engine.open(1)                      # takes the slot c gave back
    out = engine.step([sd, sa, sb], [d, a[70:71], b[69:72]],
                      [list(range(9)), [0], [0, 1, 2]]).cpu().numpy()
    assert_same_logits(out[:9], whole["d"], dtype, "d starts in a freed slot")
    assert_same_logits(out[9:10], whole["a"][70:71], dtype, "a decodes one")
    assert_same_logits(out[10:13], whole["b"][69:72], dtype, "b goes on by three")
    engine.close([sa, sb, sd])
    engine.cache.check()
    assert engine.cache.slots.held == 0


# ---- generation in bfloat16 on the fast kernels ---------------------------------------------------

@pytest.mark.parametrize("name", ["C", "D"])
def test_bfloat16_generation_chooses_the_argmax_of_a_forward_pass(name, varied_folders):
    """`generate` in bfloat16 on head sizes that the tensor-core attention kernels take, that
    is, through the decode loop that runs ahead of the host, the replayed graphs and the
    decode attention that rotates and stores on its own way: every token it chose is the
    argmax of ONE forward pass over the prompt and the tokens (the reference's test of its
    decode path, `tests/test_inference.py:140-149`), or loses to it by less than the bf16
    bound (a near tie). The weights are wide enough for the tokens to vary."""
    from helpers import BF16_RTOL
    engine = engine_for(varied_folders(name, "bfloat16"), "bfloat16")
    prompts = prompts_for(name, [5, 70, 131, 40, 64], seed=60)
    got = engine.generate([p.tolist() for p in prompts], 40, stop_at_eos=False)
    assert engine.graph_failure is None and len(engine._graphs) >= 1
    flips = 0
    for p, g in zip(prompts, got):
        assert len(g) == 40 and len(set(g.tolist())) > 8, f"tokens do not vary: {g.tolist()}"
        logits = engine.forward(np.concatenate([p, g[:-1]]))[len(p) - 1:]
        for k, token in enumerate(g.tolist()):
            best = int(logits[k].argmax())
            if token != best:
                flips += 1
                assert logits[k, best] - logits[k, token] <= BF16_RTOL * logits[k].std(), \
                    f"token {k} of a {len(p)}-token prompt: {token} chosen, {best} is the argmax"
    assert flips <= 20, f"{flips} of 200 tokens lost to a near tie: too many to be chance"
    assert engine.cache.slots.held == 0


def test_greedy_generation_of_varied_tokens(varied_folders):
    """fp32, tokens that vary (tiny-B with wide weights), through the whole loop: the plain
    model's tokens exactly, also with a stop token somewhere in the middle of each request."""
    folder = varied_folders("B", "float32")
    engine = engine_for(folder, "float32")
    config, tensors = plain.read_model_folder(folder)
    prompts = prompts_for("B", [1, 7, 30, 64], seed=61)
    want = [plain.generate(config, tensors, p, 12) for p in prompts]
    assert all(len(set(w)) > 4 for w in want)
    got = engine.generate([p.tolist() for p in prompts], 12, stop_at_eos=False)
    assert [g.tolist() for g in got] == want
    for place in (0, 3, 7, 11):
        stop = want[1][place]
        got = engine.generate([p.tolist() for p in prompts], 12, stop_token_ids=[stop])
        for g, w, e in zip(got, want, engine.endings):
            cut = w.index(stop) + 1 if stop in w else len(w)
            assert g.tolist() == w[:cut] and e.reason == ("stop" if stop in w else "length")
        assert len(got[1]) == want[1].index(stop) + 1 <= place + 1


def test_generation_stops_at_the_folders_end_of_sequence_ids(varied_folders, tmp_path):
    """With the default `stop_at_eos=True` the stop ids are those of generation_config.json
    (a number or a list) if the folder has one, else config.json's `eos_token_id`."""
    import json
    import shutil
    src = varied_folders("B", "float32")
    config, tensors = plain.read_model_folder(src)
    prompt = prompts_for("B", [7], seed=61)[0]
    free = plain.generate(config, tensors, prompt, 12)
    for eos in (free[4], [free[6], free[2]]):
        folder = tmp_path / f"eos_{eos if isinstance(eos, int) else 'list'}"
        shutil.copytree(src, folder)
        (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": eos}))
        engine = engine_for(folder, "float32")
        stops = {eos} if isinstance(eos, int) else set(eos)
        assert engine.eos_token_ids == frozenset(stops)
        out = engine.generate(prompt, 12).tolist()
        cut = min(free.index(s) for s in stops) + 1
        assert out == free[:cut] and engine.ending.reason == "stop"
        assert engine.generate(prompt, 12, stop_at_eos=False).tolist() == free
    # without the file: config.json's ids (tiny-B: 11 and 13)
    assert engine_for(src, "float32").eos_token_ids == frozenset({11, 13})


# ---- the diagnostics: hidden states, the cache read back, the footprint -----------------------------

@pytest.mark.parametrize("name", ["A", "B"])
def test_hidden_states_match_the_reference_models(name, engines, model_folders):
    """`forward(ids, capture_hidden_states=True)`: the embedding's output, the stream after
    each layer but the last, the last after the final norm, compared layer by layer with the
    plain model and, for the layers it stored, with what the reference's own float64 model
    computed (`tests/golden/`)."""
    from pathlib import Path
    gold = np.load(Path(__file__).parent / "golden" / f"tiny_{name}.npz")
    engine = engines(name, "float32")
    config, tensors = plain.read_model_folder(model_folders(name, "float32"))
    ids = gold["ids"]
    logits, states = engine.forward(ids, capture_hidden_states=True)
    want = plain.hidden_states(config, tensors, ids)
    assert states.shape == (config["num_hidden_layers"] + 1, len(ids), config["hidden_size"])
    for i, w in enumerate(want):
        assert np.abs(states[i] - w).max() <= FP32_RTOL_STATES * np.abs(w).max(), f"state {i}"
    keep = gold["positions"]
    np.testing.assert_allclose(states[1][keep], gold["mid_hidden"], rtol=0,
                               atol=FP32_RTOL_STATES * np.abs(gold["mid_hidden"]).max())
    np.testing.assert_allclose(states[-1][keep], gold["final_hidden"], rtol=0,
                               atol=FP32_RTOL_STATES * np.abs(gold["final_hidden"]).max())
    np.testing.assert_array_equal(logits, engine.forward(ids))     # capturing changes nothing


FP32_RTOL_STATES = 2e-5      # as for logits: of the largest magnitude of the compared state


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D", "W"])
def test_the_cache_holds_the_plain_models_keys_and_values(name, dtype, engines, model_folders):
    """`cached_kv` reads the blocks of a prefilled sequence back: rotated keys and values of
    every layer and position against the plain model's. A wrong block in ONE layer shows
    here by its layer and position, not only at the logits."""
    engine = engines(name, dtype)
    config, tensors = plain.read_model_folder(model_folders(name, stored(dtype)))
    ids = prompts_for(name, [150], seed=80)[0]
    keys, values = engine.cached_kv(ids)
    want_k, want_v = plain.cache_contents(config, tensors, ids)
    assert keys.shape == want_k.shape and values.shape == want_v.shape
    tol = 2e-5 if dtype == "float32" else 2e-2
    for layer in range(config["num_hidden_layers"]):
        window = plain.layer_window(config, layer)
        first = 0 if window is None else (max(0, len(ids) - window + 1) // 64) * 64
        assert np.isnan(keys[layer, :first]).all()           # blocks the window gave back
        for got, want, what in ((keys, want_k, "keys"), (values, want_v, "values")):
            diff = np.abs(got[layer, first:] - want[layer, first:])
            assert diff.max() <= tol * np.abs(want[layer]).max(), \
                f"{what} of layer {layer}: position {np.unravel_index(diff.argmax(), diff.shape)[0] + first}"
    assert engine.cache.slots.held == 0


def test_footprint_counts_weights_and_cache(model_folders):
    engine = engine_for(model_folders("B", "bfloat16"), "bfloat16", max_tokens=640)
    before = engine.footprint()
    assert before["kv_cache"] == 0 and before["weights"] == engine.model.arena.nbytes > 0
    engine.forward([1, 2, 3])
    after = engine.footprint()
    # three layers of one KV head of 32: keys and values, 10 blocks of 64, two bytes each
    assert after["kv_cache"] == 3 * 2 * 10 * 64 * 32 * 2
    assert 0 < after["device_free"] <= after["device_total"]


def test_allocation_failures_leave_the_engine_as_it_was(model_folders, monkeypatch):
    """An allocation that fails while the weights or the cache are built raises the typed
    error and leaves no half-built state (`tests/test_emergency_downgrade.py:40-54` of the
    reference injects its failures on the host in the same way)."""
    from semantic_aware_adaptive_kv_cache_precision_b200 import Engine, OutOfDeviceMemory
    folder = model_folders("A", "float32")
    engine = Engine(folder, dtype="float32", max_tokens=256)
    real_empty, real_zeros = torch.empty, torch.zeros
    state = {"fail": True}

    def empty(*args, **kwargs):
        if state["fail"] and kwargs.get("dtype") == torch.uint8:
            raise torch.OutOfMemoryError("injected")
        return real_empty(*args, **kwargs)

    def zeros(*args, **kwargs):
        if state["fail"] and args and isinstance(args[0], tuple) and len(args[0]) == 5:
            raise torch.OutOfMemoryError("injected")
        return real_zeros(*args, **kwargs)

    monkeypatch.setattr(torch, "empty", empty)
    monkeypatch.setattr(torch, "zeros", zeros)
    with pytest.raises(OutOfDeviceMemory, match="weights"):
        engine.load_weights()
    assert not engine._loaded and engine.model.arena is None
    with pytest.raises(RuntimeError, match="load_weights"):
        engine.forward([1, 2])
    state["fail"] = False
    engine.load_weights()
    state["fail"] = True
    with pytest.raises(OutOfDeviceMemory, match="cache"):
        engine.forward([1, 2])
    assert engine.cache is None
    state["fail"] = False
    ids = prompts_for("A", [9], seed=81)[0]
    assert_close_to_plain(engine.forward(ids), plain_logits(folder, ids), "float32", "after")


# ---- random schedules ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "W", "D"])
def test_random_schedules_give_the_logits_of_whole_prompts(name, dtype, engines):
    """Forty steps drawn at random over a pool of requests: a step may start new requests,
    feed others a piece of any length, decode others by one token and end some, all in one
    batch, in a cache that forces slots and blocks to be used again. Whatever the schedule,
    every position's logits are those of its request run alone and whole: to the bit in
    32-bit, within rounding in bfloat16 (a fault of the cache or of the batch shows as ONE
    request's rows going wrong from some step on)."""
    engine = engines(name, dtype)
    limit = {"B": 250, "W": 300, "D": 400}[name]
    rng = np.random.default_rng({"B": 1, "W": 2, "D": 3}[name])
    lengths = rng.integers(1, limit, 14).tolist()
    prompts = prompts_for(name, lengths, seed=90)
    whole = [engine.forward(p) for p in prompts]
    waiting = list(range(len(prompts)))
    live: dict[int, tuple[int, int]] = {}              # request -> (slot, tokens fed)
    steps = 0
    while waiting or live:
        steps += 1
        assert steps < 400
        room = 6 - len(live)
        starters = [waiting.pop(0) for _ in range(min(len(waiting), int(rng.integers(0, room + 1))))]
        for r, slot in zip(starters, engine.open(len(starters))):
            live[r] = (slot, 0)
        chosen = [r for r in live if rng.random() < 0.7 or live[r][1] == 0]
        if not chosen:
            continue
        slots, tokens, want, spans = [], [], [], []
        for r in chosen:
            slot, fed = live[r]
            left = len(prompts[r]) - fed
            kind = rng.random()
            count = 1 if kind < 0.4 else int(rng.integers(1, left + 1)) if kind < 0.8 else left
            count = min(count, left)
            rows = sorted(set(rng.integers(0, count, min(count, 5)).tolist() + [count - 1]))
            slots.append(slot)
            tokens.append(prompts[r][fed:fed + count])
            want.append(rows)
            spans.append((r, fed, rows))
            live[r] = (slot, fed + count)
        out = engine.step(slots, tokens, want).cpu().numpy()
        at = 0
        for r, fed, rows in spans:
            got = out[at:at + len(rows)]
            at += len(rows)
            assert_same_logits(got, whole[r][[fed + k for k in rows]], dtype,
                               f"{name} step {steps}: request {r} of {len(prompts[r])} tokens, "
                               f"rows {fed + rows[0]}..{fed + rows[-1]}")
        done = [r for r in chosen if live[r][1] == len(prompts[r])]
        if done:
            engine.close([live.pop(r)[0] for r in done])
        engine.cache.check()
    assert engine.cache.slots.held == 0 and all(g.pool.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_next_tokens_is_a_step_and_its_greedy_choice(name, dtype, varied_folders):
    """`Engine.next_tokens` (the choice inside the captured step, the tokens left where the
    next step reads them) gives what `step` followed by the greedy choice gives, step after
    step: fed with its own result (nothing copied), with a copy of it, with a batch that
    shrinks, and after another step has used the staging buffer in between."""
    from semantic_aware_adaptive_kv_cache_precision_b200 import sampling
    folder = varied_folders(name, stored(dtype))
    two = [engine_for(folder, dtype) for _ in range(2)]
    prompts = prompts_for(name, [70, 5, 130, 64], seed=5)
    greedy = sampling.SamplingParams()
    fed, slots = [], []
    for engine in two:
        s = engine.open(len(prompts))
        logits = engine.step(s, prompts)
        fed.append(sampling.choose(logits, greedy))
        slots.append(s)
    assert torch.equal(fed[0], fed[1])
    live = list(range(len(prompts)))
    history = []
    for t in range(40):
        a = two[0].next_tokens([slots[0][i] for i in live], fed[0])
        b = sampling.choose(two[1].step([slots[1][i] for i in live], device_tokens=fed[1]), greedy)
        assert torch.equal(a, b), f"step {t}: {a.tolist()} against {b.tolist()}"
        history.append(a.tolist())
        fed = [a, b]
        if t % 7 == 3:
            fed[0] = a.clone()                        # not the engine's own buffer
        if t == 10:                                   # another step uses the staging buffer
            kept = a.clone()
            (other,) = two[0].open(1)
            two[0].step([other], [prompts[0][:9]])
            two[0].close([other])
            fed[0] = kept
        if t in (15, 25):                             # a request leaves
            gone = live.pop(1)
            for engine, s in zip(two, slots):
                engine.close([s[gone]])
            keep = torch.as_tensor([j for j in range(len(live) + 1) if j != 1], device=a.device)
            fed = [f[keep] for f in fed]
    assert len({tuple(h) for h in history}) > 10      # (the tokens do vary)
    for engine, s in zip(two, slots):
        engine.close([s[i] for i in live])
        assert engine.cache.slots.held == 0

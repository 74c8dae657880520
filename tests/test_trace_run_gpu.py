"""bin/trace_run as a user runs it: a process fed one step a line, answering
`done <step>` after each. The same requests are replayed whole, with their last
32 tokens one by one, and in batches of unequal lengths one after another in a
cache that only just holds a batch (so slots and blocks are used again); all
three are compared with the plain implementation and with each other."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from conftest import ROOT, TINY, prompts_for
from helpers import assert_close_to_plain, assert_same_logits, plain_logits

pytestmark = pytest.mark.gpu


class Trace:
    """Drives one trace_run process, one step at a time."""

    def __init__(self, folder, dtype, out, max_tokens):
        self.out = Path(out)
        self.proc = subprocess.Popen(
            [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
             dtype, "--out", str(out), "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.step = 0

    def send(self, entries, end=()):
        record = {"step": self.step, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(record) + "\n")
        self.proc.stdin.flush()
        answer = self.proc.stdout.readline().strip()
        assert answer == f"done {self.step}", f"trace_run answered {answer!r}"
        wanted = sum(len(e["want"]) for e in entries)
        path = self.out / f"{self.step}.f32"
        self.step += 1
        if not wanted:
            assert not path.exists()
            return None
        data = np.fromfile(path, dtype="<f4")
        return data.reshape(wanted, -1)

    def finish(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


def entry(name, tokens, want):
    return {"id": name, "tokens": [int(t) for t in tokens], "want": list(want)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_replay_three_ways(name, dtype, model_folders, tmp_path):
    folder = model_folders(name, "float32" if dtype == "float32" else "bfloat16")
    vocab = TINY[name][0]["vocab_size"]
    lengths = {"A": [40, 97, 33, 128, 64, 50], "B": [33, 120, 250, 64, 65, 36],
               "W": [100, 290, 36, 75, 141, 200]}[name]
    prompts = prompts_for(name, lengths, seed=20)
    want = [plain_logits(folder, p) for p in prompts]
    # the cache holds one batch of three at their full lengths, rounded up to blocks
    batches = [[0, 1, 2], [3, 4, 5]]
    max_tokens = max(sum(-(-lengths[i] // 64) * 64 for i in b) for b in batches)
    trace = Trace(folder, dtype, tmp_path / "out", max_tokens)

    whole = []
    for i, p in enumerate(prompts):
        got = trace.send([entry(f"w{i}", p, range(len(p)))], end=[f"w{i}"])
        assert got.shape == (len(p), vocab)
        whole.append(got)
        assert_close_to_plain(got, want[i], dtype, f"{name} request {i} whole")

    for i, p in enumerate(prompts):
        head = len(p) - 32
        rows = [trace.send([entry(f"s{i}", p[:head], range(head))])]
        for t in range(head, len(p)):
            rows.append(trace.send([entry(f"s{i}", p[t:t + 1], [0])],
                                   end=[f"s{i}"] if t == len(p) - 1 else []))
        stepped = np.concatenate(rows)
        assert_same_logits(stepped, whole[i], dtype, f"{name} request {i}: last 32 one by one")
        assert_close_to_plain(stepped, want[i], dtype, f"{name} request {i} stepped")

    for b, members in enumerate(batches):
        # prompts go in without their last 1..12 tokens, which are then decoded; the
        # shorter tails end earlier
        tails = {i: 1 + (5 * k + 3 * b) % 12 for k, i in enumerate(members)}
        heads = {i: len(prompts[i]) - tails[i] for i in members}
        got = trace.send([entry(f"b{i}", prompts[i][:heads[i]], range(heads[i]))
                          for i in members])
        rows = {i: [] for i in members}
        at = 0
        for i in members:
            rows[i].append(got[at:at + heads[i]])
            at += heads[i]
        fed = dict(heads)
        live = list(members)
        while live:
            ending = [i for i in live if fed[i] + 1 == len(prompts[i])]
            got = trace.send([entry(f"b{i}", prompts[i][fed[i]:fed[i] + 1], [0]) for i in live],
                             end=[f"b{i}" for i in ending])
            for r, i in enumerate(live):
                rows[i].append(got[r:r + 1])
                fed[i] += 1
            live = [i for i in live if i not in ending]
        for i in members:
            batched = np.concatenate(rows[i])
            assert_same_logits(batched, whole[i], dtype, f"{name} request {i}: batch {b}")
            assert_close_to_plain(batched, want[i], dtype, f"{name} request {i} batched")

    # a step may want nothing, and an unknown id in `end` is an error that ends the run
    assert trace.send([entry("x", prompts[0][:5], [])]) is None
    assert trace.send([entry("x", prompts[0][5:6], [0])], end=["x"]).shape == (1, vocab)
    trace.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_requests_may_join_a_running_batch(name, dtype, model_folders, tmp_path):
    """A step may hold requests that start beside requests that go on by one token or by
    several: a starts with 70 tokens while b brings 5 after 64 and c one after 200. Every
    position's logits are those of the request replayed alone and whole."""
    folder = model_folders(name, "float32" if dtype == "float32" else "bfloat16")
    a, b, c = prompts_for(name, [71, 69, 201], seed=21)
    trace = Trace(folder, dtype, tmp_path / "out", 512)
    whole = {}
    for key, p in (("a", a), ("b", b), ("c", c)):
        whole[key] = trace.send([entry("w" + key, p, range(len(p)))], end=["w" + key])
    assert trace.send([entry("b", b[:64], []), entry("c", c[:200], [])]) is None
    got = trace.send([entry("a", a[:70], range(70)), entry("b", b[64:], range(5)),
                      entry("c", c[200:], [0])], end=["b", "c"])
    assert_same_logits(got[:70], whole["a"][:70], dtype, "a starts beside others")
    assert_same_logits(got[70:75], whole["b"][64:], dtype, "b goes on by five")
    assert_same_logits(got[75:], whole["c"][200:], dtype, "c goes on by one")
    got = trace.send([entry("a", a[70:], [0])], end=["a"])
    assert_same_logits(got, whole["a"][70:], dtype, "a decodes after the mixed step")
    trace.finish()


def test_trace_run_ends_with_an_error_on_a_bad_step(model_folders, tmp_path):
    folder = model_folders("A", "float32")
    trace = Trace(folder, "float32", tmp_path / "out", 256)
    trace.send([entry("a", [1, 2, 3], [2])])
    trace.proc.stdin.write(json.dumps({"step": 1, "entries": [entry("a", [4], [0])],
                                       "end": ["nobody"]}) + "\n")
    trace.proc.stdin.close()
    assert trace.proc.wait(timeout=60) != 0

"""Trace replay: given token ids go through the model step by step, logits come out.

It samples nothing and has no model code of its own: every step is one call of
`Engine.step`, the step function that generation uses, on the engine's own
cache. The nearest thing in the reference is teacher forcing on a conversation
(`Conversation.force`, `src/microinfer/engine.py:620-671`).

A trace is a stream of JSON objects, one a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries` gives each request's next tokens and the places among them whose
logits are wanted; `end` names requests that are finished after the step. A
request starts at the step that names it first; requests that start and
requests that go on (by one token or by many) may share a step. For a
step that wants something, `<out>/<step>.f32` receives the logits at the wanted
places in the order of the entries, little-endian fp32 [wanted, vocab]. After
every step the line `done <step>` is printed and flushed.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np

from .engine import Engine


class TraceError(ValueError):
    pass


class Replayer:
    def __init__(self, engine: Engine, out_dir):
        self.engine = engine
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.slot_of: dict[str, int] = {}

    def run_step(self, record: dict) -> None:
        if "step" not in record:
            raise TraceError("a step needs a 'step' field")
        step = record["step"]
        entries = record.get("entries", [])
        names = [e["id"] for e in entries]
        if len(set(names)) != len(names):
            raise TraceError(f"step {step}: a request appears twice")
        # requests not seen before start here; they may do so beside requests that go on
        # (the step function takes both in one batch)
        fresh = [n for n in names if n not in self.slot_of]
        if fresh:
            for request, slot in zip(fresh, self.engine.open(len(fresh))):
                self.slot_of[request] = slot
        wanted = 0
        if entries:
            slots = [self.slot_of[e["id"]] for e in entries]
            tokens = [np.asarray(e["tokens"], dtype=np.int64) for e in entries]
            vocab = self.engine.vocab_size
            for e, t in zip(entries, tokens):
                if t.size == 0:
                    raise TraceError(f"step {step}: request {e['id']!r} brings no tokens")
                if t.min() < 0 or t.max() >= vocab:
                    raise TraceError(f"step {step}: request {e['id']!r} has token ids outside "
                                     f"[0, {vocab})")
            want = [list(e.get("want", [])) for e in entries]
            wanted = sum(len(w) for w in want)
            logits = self.engine.step(slots, tokens, want)
            if wanted:
                data = logits.cpu().numpy().astype("<f4", copy=False)
                data.tofile(self.out_dir / f"{step}.f32")
        ended = record.get("end", [])
        unknown = [r for r in ended if r not in self.slot_of]
        if unknown:
            raise TraceError(f"step {step}: 'end' names unknown requests {unknown}")
        if ended:
            self.engine.close([self.slot_of.pop(r) for r in ended])

    def run(self, lines, report=sys.stdout) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            self.run_step(record)
            print(f"done {record['step']}", file=report, flush=True)


def main(argv=None) -> int:
    import argparse
    parser = argparse.ArgumentParser(
        prog="trace_run",
        description="Feed given token ids through a model step by step and write logits.")
    parser.add_argument("--model", required=True,
                        help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                        help="bfloat16: the serving kernels; float32: everything in true 32-bit")
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time, each request "
                             "rounded up to a multiple of 64; sizes the cache")
    args = parser.parse_args(argv)
    engine = Engine(args.model, dtype=args.dtype, max_tokens=args.max_tokens).load_weights()
    Replayer(engine, args.out).run(sys.stdin)
    return 0

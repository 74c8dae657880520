"""The command line, in the manner of the reference's tools (argparse scripts with
`--model`, `--new-tokens`, `--lengths`, `--repeat`, `--warmup`; `tools/tier_samples.py:
64-72`, `tools/throughput.py:215-238`).

    python -m semantic_aware_adaptive_kv_cache_precision_b200 generate --model DIR \
        --prompt-ids 1,2,3 --prompt-ids 4,5 --new-tokens 16 [--temperature 0.8 --seed 1]
    python -m semantic_aware_adaptive_kv_cache_precision_b200 throughput --model DIR \
        --lengths 512 2048 --repeat 3 --warmup 1
    python -m semantic_aware_adaptive_kv_cache_precision_b200 random-model --config config.json \
        --seed 0 --out DIR

Prompts are token ids; text is taken only if the model folder has a tokenizer.json and
the `tokenizers` package is installed (`src/microinfer/engine.py:1133-1146`).
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from pathlib import Path


def _ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def _engine(args):
    from .engine import Engine
    return Engine(args.model, dtype=args.dtype, max_tokens=args.max_tokens,
                  max_batch=args.max_batch).load_weights()


def cmd_generate(args) -> int:
    prompts = [_ids(p) for p in args.prompt_ids or []]
    if args.prompt_file:
        prompts += [_ids(line) for line in Path(args.prompt_file).read_text().splitlines()
                    if line.strip()]
    if not prompts and not args.prompt:
        raise SystemExit("give --prompt-ids, --prompt-file or --prompt")
    engine = _engine(args)
    if args.prompt:
        try:
            prompts += [engine.encode(p).tolist() for p in args.prompt]
        except RuntimeError as exc:             # no tokenizer.json, or no `tokenizers` package
            raise SystemExit(f"{exc}; give token ids with --prompt-ids") from None
    out = engine.generate(prompts, args.new_tokens, stop_at_eos=not args.ignore_eos,
                          temperature=args.temperature, seed=args.seed)
    for i, (tokens, ending) in enumerate(zip(out, engine.endings)):
        record = {"request": i, "tokens": tokens.tolist(), "ending": ending.state,
                  "reason": ending.reason, "positions": ending.positions}
        if args.prompt:
            record["text"] = engine.decode(tokens.tolist())
        print(json.dumps(record))
    return 0


def cmd_throughput(args) -> int:
    """Prefill and decode tokens a second on random token ids, as the reference
    measures them (`tools/throughput.py:66-73, 258-293`): median of `--repeat` after
    `--warmup`; prefill = time of generate(prompt, 1); decode = (time of 33 tokens -
    time of 1 token) / 32."""
    import numpy as np
    engine = _engine(args)
    rng = np.random.default_rng(0)
    steps = 32

    def timed(fn):
        runs = []
        for i in range(args.warmup + args.repeat):
            began = time.perf_counter()
            fn()
            if i >= args.warmup:
                runs.append(time.perf_counter() - began)
        return statistics.median(runs)

    for length in args.lengths:
        prompts = [rng.integers(0, engine.vocab_size, length).tolist()
                   for _ in range(args.batch)]
        first = timed(lambda: engine.generate(prompts, 1, stop_at_eos=False))
        more = timed(lambda: engine.generate(prompts, steps + 1, stop_at_eos=False))
        print(json.dumps({"length": length, "batch": args.batch,
                          "prefill_tokens_per_second": args.batch * length / first,
                          "decode_tokens_per_second": args.batch * steps / max(more - first, 1e-9)}))
    return 0


def cmd_random_model(args) -> int:
    from .weights import write_random_model
    config = json.loads(Path(args.config).read_text())
    folder = write_random_model(args.out, config, args.seed, dtype=args.stored_dtype)
    print(folder)
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="semantic_aware_adaptive_kv_cache_precision_b200",
                                     description=__doc__.splitlines()[0])
    sub = parser.add_subparsers(dest="command", required=True)

    def common(p):
        p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
        p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
        p.add_argument("--max-tokens", type=int, default=16384,
                       help="cache positions over all live sequences")
        p.add_argument("--max-batch", type=int, default=64)

    g = sub.add_parser("generate", help="generate tokens for one or more prompts")
    common(g)
    g.add_argument("--prompt-ids", action="append", help="token ids, comma or space separated; "
                   "repeat for a batch")
    g.add_argument("--prompt-file", help="file with one prompt of token ids per line")
    g.add_argument("--prompt", action="append", help="text (needs tokenizer.json)")
    g.add_argument("--new-tokens", type=int, default=64)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--ignore-eos", action="store_true", help="do not stop at end-of-sequence ids")
    g.set_defaults(run=cmd_generate)

    t = sub.add_parser("throughput", help="prefill and decode tokens a second on random ids")
    common(t)
    t.add_argument("--lengths", type=int, nargs="+", default=[512, 2048, 8192])
    t.add_argument("--repeat", type=int, default=3)
    t.add_argument("--warmup", type=int, default=1)
    t.add_argument("--batch", type=int, default=1)
    t.set_defaults(run=cmd_throughput)

    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--stored-dtype", choices=["bfloat16", "float32", "float16"], default=None)
    r.set_defaults(run=cmd_random_model)

    args = parser.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())

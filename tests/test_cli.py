"""The command line as a user runs it: `python -m semantic_aware_adaptive_kv_cache_precision_b200
generate | throughput | random-model` as child processes, their JSON lines parsed; and text in
and out through a tokenizer.json made here with the `tokenizers` package (no network)."""

import json
import subprocess
import sys

import numpy as np
import pytest

import plain_model as plain
from conftest import ROOT, TINY_B, prompts_for

MODULE = "semantic_aware_adaptive_kv_cache_precision_b200"


def run(*args, timeout=600):
    out = subprocess.run([sys.executable, "-m", MODULE, *args], capture_output=True, text=True,
                         cwd=str(ROOT), timeout=timeout)
    assert out.returncode == 0, out.stderr[-2000:]
    return [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")], out


def test_random_model_writes_a_folder_that_reads_back(tmp_path):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(dict(TINY_B, initializer_range=0.1)))
    _, out = run("random-model", "--config", str(config), "--seed", "5", "--out",
                 str(tmp_path / "m"), "--stored-dtype", "float32")
    assert out.stdout.strip().endswith("m")
    cfg, tensors = plain.read_model_folder(tmp_path / "m")
    assert cfg["architectures"] == ["Qwen2ForCausalLM"] and cfg["torch_dtype"] == "float32"
    assert tensors["lm_head.weight"].shape == (1000, 192)
    assert abs(tensors["lm_head.weight"].std() - 0.1) < 0.01


@pytest.mark.gpu
def test_generate_and_throughput_commands(varied_folders):
    folder = varied_folders("B", "float32")
    config, tensors = plain.read_model_folder(folder)
    prompts = prompts_for("B", [7, 30], seed=61)
    want = [plain.generate(config, tensors, p, 8) for p in prompts]
    records, _ = run("generate", "--model", str(folder), "--dtype", "float32", "--ignore-eos",
                     "--prompt-ids", ",".join(map(str, prompts[0])),
                     "--prompt-ids", " ".join(map(str, prompts[1])), "--new-tokens", "8")
    assert [r["request"] for r in records] == [0, 1]
    assert [r["tokens"] for r in records] == want
    assert all(r["ending"] == "complete" and r["reason"] == "length" for r in records)
    assert [r["positions"] for r in records] == [len(p) + 7 for p in prompts]
    # temperature: reproducible for a seed, different for another
    def sampled(seed):
        return run("generate", "--model", str(folder), "--dtype", "float32", "--ignore-eos",
                   "--prompt-ids", ",".join(map(str, prompts[0])), "--new-tokens", "8",
                   "--temperature", "0.9", "--seed", str(seed))[0][0]["tokens"]
    first = sampled(3)
    assert first == plain.generate(config, tensors, prompts[0], 8, temperature=0.9, seed=3)
    assert first != sampled(4)
    records, _ = run("throughput", "--model", str(folder), "--lengths", "64", "100",
                     "--repeat", "1", "--warmup", "1", "--batch", "2")
    assert [r["length"] for r in records] == [64, 100] and all(r["batch"] == 2 for r in records)
    assert all(r["prefill_tokens_per_second"] > 0 and r["decode_tokens_per_second"] > 0
               for r in records)


def word_tokenizer(folder, vocab_size):
    """A tokenizer.json of whole words w0, w1, ...: word i is token i."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    vocab = {f"w{i}": i for i in range(vocab_size - 1)}
    vocab["[UNK]"] = vocab_size - 1
    tokenizer = Tokenizer(WordLevel(vocab, unk_token="[UNK]"))
    tokenizer.pre_tokenizer = Whitespace()
    tokenizer.save(str(folder / "tokenizer.json"))


@pytest.mark.gpu
def test_text_goes_in_and_out_through_the_folders_tokenizer(varied_folders, tmp_path):
    import shutil
    from semantic_aware_adaptive_kv_cache_precision_b200 import Engine
    src = varied_folders("B", "float32")
    bare = Engine(src, dtype="float32", max_tokens=512).load_weights()
    with pytest.raises(RuntimeError, match="no tokenizer.json"):
        bare.generate("w1 w2", 2)
    folder = tmp_path / "with_tokenizer"
    shutil.copytree(src, folder)
    word_tokenizer(folder, 1000)
    engine = Engine(folder, dtype="float32", max_tokens=512).load_weights()
    ids = [5, 17, 3, 900]
    text = " ".join(f"w{i}" for i in ids)
    assert engine.encode(text).tolist() == ids and engine.encode(text).dtype == np.int32
    assert engine.decode(ids) == text
    from_ids = engine.generate(ids, 6, stop_at_eos=False).tolist()
    assert engine.generate(text, 6, stop_at_eos=False).tolist() == from_ids
    both = engine.generate([text, [1, 2]], 6, stop_at_eos=False)
    assert both[0].tolist() == from_ids
    records, _ = run("generate", "--model", str(folder), "--dtype", "float32", "--ignore-eos",
                     "--prompt", text, "--new-tokens", "6")
    assert records[0]["tokens"] == from_ids
    assert records[0]["text"] == engine.decode(from_ids)

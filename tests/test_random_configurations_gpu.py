"""Configurations drawn at random over what config.json allows: the engine gives the plain
model's logits or refuses the configuration with a clear error, never a wrong result.

The five fixed tiny configurations pin the kernels' paths; this file walks the space between
them. Each seed draws head sizes in steps of 16 from 16 to 256 (and 24 and 272, which the
attention kernels refuse), one to five key/value heads with one to eight query heads each, a
hidden size that is the heads' width or one of its own (34 to 1,030: no power of two, some no
multiple of 8, so that the products fall to the library's kernels), intermediate sizes from
24 to 4,104 (odd ones too), vocabularies from 37 to 40,001, one to three layers, the three
values of eps, tied and untied heads, and a window of 5 to 130 positions on some, all or none
of the layers. Every configuration then runs whole prompts (1, a few, some 100 and some 300
tokens), the last 20 tokens of one prompt one by one, and the four prompts as one unequal
batch that decodes its last five tokens with the shorter requests ending earlier, in 32-bit
and in bfloat16, with freed cache blocks poisoned. Widths stay at or below 2,048 so that the
small tests' bfloat16 bound holds (wider rows carry more rounding noise; the real widths have
a test of their own with a criterion made for them)."""

import json

import numpy as np
import pytest

from helpers import assert_close_to_plain, plain_logits

SEEDS = list(range(32))
REFUSED_HEAD_SIZES = (24, 272)


def draw_configuration(seed: int):
    rng = np.random.default_rng(7000 + seed)
    while True:
        head_dim = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 160, 176, 192, 208,
                                   224, 240, 256, 24, 272]))
        kv_heads = int(rng.choice([1, 2, 3, 4, 5]))
        heads = kv_heads * int(rng.choice([1, 2, 3, 4, 6, 7, 8]))
        if heads * head_dim <= 2048:
            break
    own_hidden = bool(rng.integers(0, 2))
    hidden = int(rng.choice([34, 40, 50, 66, 72, 100, 136, 200, 264, 520, 1030])) \
        if own_hidden else heads * head_dim
    layers = int(rng.integers(1, 4))
    config = {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
        "num_hidden_layers": layers, "hidden_size": hidden, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads,
        "intermediate_size": int(rng.choice([24, 33, 88, 99, 100, 101, 176, 200, 328, 520, 1000,
                                             4104])),
        "vocab_size": int(rng.choice([37, 100, 257, 1000, 3001, 40001])),
        "max_position_embeddings": 1024, "rope_theta": float(rng.choice([1e4, 5e4, 1e6])),
        "rms_norm_eps": float(rng.choice([1e-6, 3e-6, 1e-5])),
        "tie_word_embeddings": bool(rng.integers(0, 2)), "hidden_act": "silu",
        "torch_dtype": "float32", "use_sliding_window": bool(rng.integers(0, 2)),
        "eos_token_id": 1,
    }
    if own_hidden:
        config["head_dim"] = head_dim
    if config["use_sliding_window"]:
        config["sliding_window"] = int(rng.choice([5, 64, 70, 130]))
        config["max_window_layers"] = int(rng.integers(0, layers + 1))
    return config, head_dim, rng


def test_the_draws_cover_the_space():
    """(what the file's first paragraph promises of its seeds)"""
    drawn = [draw_configuration(s) for s in SEEDS]
    configs = [c for c, _, _ in drawn]
    assert any(d in REFUSED_HEAD_SIZES for _, d, _ in drawn)
    assert len({d for _, d, _ in drawn}) >= 8
    assert any(c["hidden_size"] % 8 for c in configs)
    assert any(c["intermediate_size"] % 2 for c in configs)
    assert any(c["use_sliding_window"] and 0 < c["max_window_layers"] < c["num_hidden_layers"]
               for c in configs)
    assert {c["tie_word_embeddings"] for c in configs} == {True, False}
    assert any(c["num_attention_heads"] // c["num_key_value_heads"] == 7 for c in configs)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", SEEDS)
def test_a_random_configuration_gives_the_plain_models_logits_or_is_refused(seed, dtype, tmp_path):
    from semantic_aware_adaptive_kv_cache_precision_b200 import Engine, write_random_model
    config, head_dim, rng = draw_configuration(seed)
    what = (f"seed {seed}: head size {head_dim}, {config['num_attention_heads']} heads over "
            f"{config['num_key_value_heads']}, hidden {config['hidden_size']}, intermediate "
            f"{config['intermediate_size']}, vocabulary {config['vocab_size']}")
    if head_dim in REFUSED_HEAD_SIZES:
        # (refused before any weight is read: the folder needs no more than its config.json)
        (tmp_path / "model").mkdir()
        (tmp_path / "model" / "config.json").write_text(json.dumps(config))
        with pytest.raises(ValueError, match=f"head_dim {head_dim}"):
            Engine(tmp_path / "model", dtype=dtype, max_tokens=1024).load_weights()
        with pytest.raises(ValueError, match=f"head_dim {head_dim}"):
            write_random_model(tmp_path / "other", dict(config), seed, dtype=dtype)
        return
    folder = write_random_model(tmp_path / "model", dict(config), seed, dtype=dtype)
    engine = Engine(folder, dtype=dtype, poison_freed=True, max_tokens=2048).load_weights()
    try:
        lengths = [1, int(rng.integers(2, 64)), int(rng.integers(64, 200)),
                   int(rng.integers(200, 420))]
        prompts = [rng.integers(0, config["vocab_size"], n).astype(np.int64) for n in lengths]
        wants = [plain_logits(folder, p) for p in prompts]
        for p, want in zip(prompts, wants):
            assert_close_to_plain(engine.forward(p), want, dtype, f"{what}; whole, {len(p)} tokens")

        p, want = prompts[2], wants[2]
        (slot,) = engine.open(1)
        head = len(p) - 20
        rows = [engine.step([slot], [p[:head]], [list(range(head))]).cpu().numpy()]
        for t in range(head, len(p)):
            rows.append(engine.step([slot], [p[t:t + 1]]).cpu().numpy())
        engine.close([slot])
        assert_close_to_plain(np.concatenate(rows), want, dtype, f"{what}; last 20 one by one")

        fed = [max(1, len(q) - 5) for q in prompts]
        slots = engine.open(len(prompts))
        out = engine.step(slots, [q[:n] for q, n in zip(prompts, fed)],
                          [list(range(n)) for n in fed]).cpu().numpy()
        got, at = [], 0
        for n in fed:
            got.append([out[at:at + n]])
            at += n
        live = list(range(len(prompts)))
        while live:
            done = [i for i in live if fed[i] == len(prompts[i])]
            if done:
                engine.close([slots[i] for i in done])       # the shorter requests end earlier
                live = [i for i in live if i not in done]
                engine.cache.check()
                continue
            out = engine.step([slots[i] for i in live],
                              [prompts[i][fed[i]:fed[i] + 1] for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1])
                fed[i] += 1
        for i, want in enumerate(wants):
            assert_close_to_plain(np.concatenate(got[i]), want, dtype, f"{what}; batched, request {i}")
        assert engine.cache.slots.held == 0
        assert all(g.pool.held == 0 for g in engine.cache.groups)
    finally:
        engine.release()

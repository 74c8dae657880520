"""The plain implementation against the reference's own float64 model, and its
parts against their definitions. No GPU.

`tests/golden/tiny_*.npz` hold what the reference's `forward64`
(`tools/conditioning.py:43-82`) computed on the tiny random checkpoints; the
script beside them made them. If the reference checkout is present the
comparison is also made afresh."""

import hashlib
import os
from pathlib import Path

import numpy as np
import pytest

import plain_model as plain
from conftest import TINY, prompts_for

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_float64_model(name, model_folders):
    gold = np.load(GOLDEN / f"tiny_{name}.npz")
    folder = model_folders(name, "float32")
    digest = hashlib.sha256((folder / "model.safetensors").read_bytes()).hexdigest()
    assert digest == str(gold["sha256"]), \
        "the random-weights mode no longer writes the checkpoint the golden file was made from"
    config, tensors = plain.read_model_folder(folder)
    ids = gold["ids"]
    states = plain.hidden_states(config, tensors, ids)
    keep = gold["positions"]
    np.testing.assert_allclose(states[1][keep], gold["mid_hidden"], rtol=0, atol=2e-7)
    np.testing.assert_allclose(states[-1][keep], gold["final_hidden"], rtol=0, atol=2e-6)
    logits = plain.forward(config, tensors, ids)
    np.testing.assert_allclose(logits[keep], gold["logits"], rtol=0, atol=2e-6)


# the reference's checkout, if there is one beside this repository (or where
# MICROINFER_REFERENCE points)
REFERENCE = Path(os.environ.get("MICROINFER_REFERENCE",
                                Path(__file__).resolve().parents[2] / "reference"))


@pytest.mark.skipif(not (REFERENCE / "tools" / "conditioning.py").is_file(),
                    reason="no reference checkout")
def test_plain_matches_reference_run_afresh(model_folders):
    import sys
    sys.path.insert(0, str(GOLDEN))
    from make_golden import reference_forward64
    ModelConfig, read_tensor, forward64 = reference_forward64(REFERENCE)
    config, _ = TINY["A"]
    folder = model_folders("A", "float32")
    ids = prompts_for("A", [23], seed=5)[0]
    ref = forward64(ModelConfig.from_dict("a", dict(config)), folder / "model.safetensors", ids, 0.0)
    cfg, tensors = plain.read_model_folder(folder)
    mine = plain.hidden_states(cfg, tensors, ids)
    for a, b in zip(mine, ref):
        np.testing.assert_allclose(a, b, rtol=0, atol=1e-12)


def test_rms_norm_definition():
    rng = np.random.default_rng(0)
    x, w = rng.standard_normal((3, 10)), rng.standard_normal(10)
    y = plain.rms_norm(x, w, 1e-3)
    for r in range(3):
        np.testing.assert_allclose(y[r], x[r] / np.sqrt(np.mean(x[r] ** 2) + 1e-3) * w)


def test_rotation_keeps_length_and_is_relative():
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal((1, 1, 16)), rng.standard_normal((1, 1, 16))
    dots = []
    for shift in (0, 9):
        cq, sq = plain.rope_angles([5 + shift], 16, 1e4)
        ck, sk = plain.rope_angles([2 + shift], 16, 1e4)
        rq, rk = plain.rotate_half(q, cq, sq), plain.rotate_half(k, ck, sk)
        np.testing.assert_allclose(np.linalg.norm(rq), np.linalg.norm(q))
        dots.append(float((rq * rk).sum()))
    np.testing.assert_allclose(dots[0], dots[1], rtol=1e-12)
    c0, s0 = plain.rope_angles([0], 16, 1e4)
    np.testing.assert_array_equal(plain.rotate_half(q, c0, s0), q)


def test_causal_mask_and_window():
    m = plain.causal_mask(5)
    assert m[2].tolist() == [True, True, True, False, False]
    w = plain.causal_mask(6, window=2)
    assert w[4].tolist() == [False, False, False, True, True, False]
    assert w[0].tolist() == [True, False, False, False, False, False]


def test_first_position_attends_only_itself():
    config, _ = TINY["A"]
    rng = np.random.default_rng(2)
    h, a, g, d = 64, 4, 2, 16
    w = {"q_proj.weight": rng.standard_normal((a * d, h)), "q_proj.bias": rng.standard_normal(a * d),
         "k_proj.weight": rng.standard_normal((g * d, h)), "k_proj.bias": rng.standard_normal(g * d),
         "v_proj.weight": rng.standard_normal((g * d, h)), "v_proj.bias": rng.standard_normal(g * d),
         "o_proj.weight": np.eye(h)}
    x = rng.standard_normal((4, h))
    out = plain.attention(x, w, a, g, d, 1e4, np.arange(4))
    v0 = (x[0] @ w["v_proj.weight"].T + w["v_proj.bias"]).reshape(g, d)
    np.testing.assert_allclose(out[0].reshape(a, d), np.repeat(v0, a // g, axis=0), atol=1e-12)
    # changing a later token changes no earlier output
    x2 = x.copy()
    x2[3] += 1.0
    out2 = plain.attention(x2, w, a, g, d, 1e4, np.arange(4))
    np.testing.assert_array_equal(out[:3], out2[:3])


def test_greedy_ties_and_nan():
    assert plain.greedy(np.array([1.0, 3.0, 3.0, 2.0])) == 1
    assert plain.greedy(np.array([np.nan, 0.5, np.nan])) == 1
    assert plain.greedy(np.array([np.nan, np.nan])) == 2


def test_gumbel_noise_is_keyed_and_gumbel():
    a = plain.gumbel_noise(3, 0, 0, 4096)
    assert a.dtype == np.float32 and np.isfinite(a).all()
    np.testing.assert_array_equal(a, plain.gumbel_noise(3, 0, 0, 4096))
    for other in ((4, 0, 0), (3, 1, 0), (3, 0, 1)):
        assert not np.array_equal(a, plain.gumbel_noise(*other, 4096))
    np.testing.assert_array_equal(a[:100], plain.gumbel_noise(3, 0, 0, 100))
    big = plain.gumbel_noise(9, 2, 5, 200000)
    assert abs(big.mean() - 0.5772) < 0.02 and abs(big.var() - np.pi ** 2 / 6) < 0.05


def test_sampling_follows_the_distribution():
    logits = np.log(np.array([0.5, 0.3, 0.2], dtype=np.float32))
    draws = [plain.sample(logits, 1.0, 7, r, 0) for r in range(4000)]
    freq = np.bincount(draws, minlength=3) / 4000
    assert np.abs(freq - [0.5, 0.3, 0.2]).max() < 0.03
    assert plain.sample(logits, 0.0, 7, 0, 0) == 0


def test_generate_stops_and_keeps_the_stop_token(model_folders):
    config, tensors = plain.read_model_folder(model_folders("A", "float32"))
    prompt = prompts_for("A", [5])[0]
    full = plain.generate(config, tensors, prompt, 6)
    assert len(full) == 6
    stopped = plain.generate(config, tensors, prompt, 6, stop_token_ids={full[2]})
    assert stopped == full[:full.index(full[2]) + 1]
    assert plain.generate(config, tensors, prompt, 0) == []

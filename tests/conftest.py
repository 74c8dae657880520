"""Shared fixtures: the tiny configurations, model folders with random weights
(made in a temporary folder), and the `gpu` marker."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny Qwen2 configurations that differ in every size and option, and a third
# with a window on its later layers.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "intermediate_size": 176, "vocab_size": 512,
    "max_position_embeddings": 128, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "hidden_act": "silu", "torch_dtype": "float32",
    "use_sliding_window": False, "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6,
    "num_key_value_heads": 1, "intermediate_size": 352, "vocab_size": 1000,
    "max_position_embeddings": 256, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "float32",
    "use_sliding_window": False, "eos_token_id": [11, 13],
}
TINY_W = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 4, "hidden_size": 96, "num_attention_heads": 2,
    "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 200, "vocab_size": 301,
    "max_position_embeddings": 512, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": True, "hidden_act": "silu", "torch_dtype": "float32",
    "use_sliding_window": True, "sliding_window": 70, "max_window_layers": 1,
    "eos_token_id": 5,
}
# head sizes that the bf16 tensor-core attention kernels take: 64 with a window, and
# Qwen2.5's own 128 with 6 query heads per KV head
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 2,
    "num_key_value_heads": 1, "intermediate_size": 208, "vocab_size": 257,
    "max_position_embeddings": 1024, "rope_theta": 20000.0, "rms_norm_eps": 2e-6,
    "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "float32",
    "use_sliding_window": True, "sliding_window": 130, "max_window_layers": 2,
    "eos_token_id": 3,
}
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 384, "num_attention_heads": 12,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 320, "vocab_size": 400,
    "max_position_embeddings": 2048, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "hidden_act": "silu", "torch_dtype": "float32",
    "use_sliding_window": False, "eos_token_id": 9,
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "W": (TINY_W, 2), "C": (TINY_C, 3), "D": (TINY_D, 4)}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (fp32 and bf16 copies)."""
    from semantic_aware_adaptive_kv_cache_precision_b200 import write_random_model
    root = tmp_path_factory.mktemp("models")
    made = {}

    def get(name: str, dtype: str = "float32") -> Path:
        key = (name, dtype)
        if key not in made:
            config, seed = TINY[name]
            made[key] = write_random_model(root / f"tiny_{name}_{dtype}", dict(config), seed,
                                           dtype=dtype)
        return made[key]

    return get


@pytest.fixture(scope="session")
def varied_folders(tmp_path_factory):
    """The tiny configurations with weights drawn five times as wide (`initializer_range`
    0.1): with the usual 0.02 a tied model repeats one token for ever, which makes "the
    engine generates the plain model's tokens" say little; these generate varied tokens."""
    from semantic_aware_adaptive_kv_cache_precision_b200 import write_random_model
    root = tmp_path_factory.mktemp("varied")
    made = {}

    def get(name: str, dtype: str = "float32") -> Path:
        key = (name, dtype)
        if key not in made:
            config, seed = TINY[name]
            made[key] = write_random_model(root / f"varied_{name}_{dtype}",
                                           dict(config, initializer_range=0.1), seed,
                                           dtype=dtype)
        return made[key]

    return get


def prompts_for(name: str, lengths, seed: int = 0):
    config, _ = TINY[name]
    rng = np.random.default_rng(seed + 100)
    return [rng.integers(0, config["vocab_size"], n).astype(np.int64) for n in lengths]

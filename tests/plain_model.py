"""A plain, slow Qwen2 dense decoder in NumPy float64: the yardstick of the tests.

Whole sequences only: no cache, no batching, no step function. One function for
each part of the model, written from the formulas of the MicroInfer reference
(`src/microinfer/model.py`, `src/core_kernels/*.cu`, `tools/conditioning.py`);
each function cites the lines it restates. Nothing here imports the package
under test, and the package imports nothing from here.

The reference computes in fp16 storage with fp32 accumulation; this file
computes everything in float64, which is what its own float64 model
(`tools/conditioning.py:43-82`) does. `tests/golden/` holds that model's output
on a tiny random checkpoint, and `tests/test_plain_model.py` checks this file
against it.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

# --------------------------------------------------------------------------
# Reading a model folder (own reader: shares nothing with the package's loader)
# --------------------------------------------------------------------------


def read_safetensors(path) -> dict[str, np.ndarray]:
    """Every tensor of one safetensors file as float64 (integers stay integers).

    Layout as the reference reads it (`src/microinfer/weights.py:51-58`): an
    8-byte little-endian header length, a JSON header with `dtype`, `shape` and
    `data_offsets` for each name, then the data. bf16 is the upper half of an
    fp32 (`src/microinfer/weights.py:31-36`).
    """
    blob = Path(path).read_bytes()
    (size,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + size])
    data = memoryview(blob)[8 + size:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        kind = meta["dtype"]
        if kind == "F32":
            arr = raw.view(np.float32).astype(np.float64)
        elif kind == "F16":
            arr = raw.view(np.float16).astype(np.float64)
        elif kind == "BF16":
            arr = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif kind == "I32":
            arr = raw.view(np.int32).copy()
        elif kind == "I64":
            arr = raw.view(np.int64).copy()
        else:
            raise ValueError(f"{name}: dtype {kind} is not read here")
        out[name] = arr.reshape(meta["shape"])
    return out


def read_model_folder(folder):
    """(config dict, tensors) of a folder with config.json and model.safetensors."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    return config, read_safetensors(folder / "model.safetensors")


# --------------------------------------------------------------------------
# The parts
# --------------------------------------------------------------------------


def embed(table: np.ndarray, ids) -> np.ndarray:
    """`x[t, :] = table[ids[t], :]`, no scale and nothing added
    (`src/microinfer/model.py:363`, `src/core_kernels/embed.cu:27-43`)."""
    return table[np.asarray(ids, dtype=np.int64)]


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """`x * rsqrt(mean(x^2) + eps) * w`: the weight multiplies directly, not as
    `1 + w` (`src/core_kernels/rmsnorm.cu:43-48, 75, 79-83`)."""
    scale = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return x * scale * weight


def linear(x: np.ndarray, weight: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """`y = x W^T (+ b)` with W stored `(out, in)` row-major
    (`src/core_kernels/linear.cu:85-118`)."""
    y = x @ weight.T
    return y if bias is None else y + bias


def rope_angles(positions, head_dim: int, theta: float) -> tuple[np.ndarray, np.ndarray]:
    """cos and sin of `pos * theta^(-2j/head_dim)` for `j < head_dim/2`, formed in
    float64 (`src/core_kernels/include/microinfer/rope_angle.cuh:15-21`)."""
    j = np.arange(head_dim // 2, dtype=np.float64)
    inv_freq = np.power(float(theta), -2.0 * j / head_dim)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    return np.cos(angle), np.sin(angle)


def rotate_half(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Rotate-half pairing `j <-> j + d/2` on `x[token, head, d]`:
    `out[j] = x[j] cos - x[j+d/2] sin`, `out[j+d/2] = x[j+d/2] cos + x[j] sin`
    (`src/core_kernels/rope.cu:32-54`)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def causal_mask(n: int, window: int | None = None) -> np.ndarray:
    """True where query i may see key j: `j <= i`, the reference's only mask
    (`src/core_kernels/attention.cu:498-510`). With `window` w (Qwen2's
    `sliding_window` key, which the reference never turns on), additionally
    `i - j < w`."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    seen = j <= i
    if window is not None:
        seen &= (i - j) < window
    return seen


def softmax(scores: np.ndarray) -> np.ndarray:
    """Softmax over the last axis, the maximum taken out first
    (`src/core_kernels/attention.cu:541-657`: running maximum and sum)."""
    m = scores.max(axis=-1, keepdims=True)
    e = np.exp(scores - m)
    return e / e.sum(axis=-1, keepdims=True)


def attention(x, w: dict, heads: int, kv_heads: int, head_dim: int, theta: float,
              positions, window: int | None = None) -> np.ndarray:
    """Grouped-query causal self-attention of one whole sequence `x[n, hidden]`.

    q, k, v have a bias, o has none; q and k are rotated; query head h reads KV
    head `h // (heads / kv_heads)`; scores are scaled by `1/sqrt(head_dim)`
    (`src/microinfer/model.py:375-387`, `src/core_kernels/attention.cu:1009`).
    The reference adds the key's bias after rotation inside attention
    (`src/core_kernels/attention.cu:104-116`); rotation is linear, so this is
    the same as `k = rope(x Wk^T + bk)`, which is how its float64 model has it
    (`tools/conditioning.py:70-71`).
    """
    n = x.shape[0]
    group = heads // kv_heads
    cos, sin = rope_angles(positions, head_dim, theta)
    q = linear(x, w["q_proj.weight"], w["q_proj.bias"]).reshape(n, heads, head_dim)
    k = linear(x, w["k_proj.weight"], w["k_proj.bias"]).reshape(n, kv_heads, head_dim)
    v = linear(x, w["v_proj.weight"], w["v_proj.bias"]).reshape(n, kv_heads, head_dim)
    q, k = rotate_half(q, cos, sin), rotate_half(k, cos, sin)
    seen = causal_mask(n, window)
    out = np.empty((n, heads, head_dim))
    for h in range(heads):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].T) / np.sqrt(head_dim)
        scores = np.where(seen, scores, -np.inf)
        out[:, h, :] = softmax(scores) @ v[:, g, :]
    return linear(out.reshape(n, heads * head_dim), w["o_proj.weight"])


def swiglu_mlp(x, w: dict) -> np.ndarray:
    """`down( silu(gate(x)) * up(x) )`, silu written `g / (1 + exp(-g))`
    (`src/microinfer/model.py:392-396`, `src/core_kernels/swiglu.cu:26-38`)."""
    gate = linear(x, w["gate_proj.weight"])
    up = linear(x, w["up_proj.weight"])
    with np.errstate(over="ignore"):
        act = gate / (1.0 + np.exp(-gate)) * up
    return linear(act, w["down_proj.weight"])


def layer_window(config: dict, layer: int) -> int | None:
    """The window of one layer from Qwen2's own keys: with `use_sliding_window`,
    layers from `max_window_layers` on see the last `sliding_window` keys. The
    reference's cards have it off and its kernels never read these keys
    (`src/microinfer/model_cards/qwen2.5-1.5b-instruct.json`)."""
    if not config.get("use_sliding_window", False):
        return None
    if layer < config.get("max_window_layers", config["num_hidden_layers"]):
        return None
    return config.get("sliding_window")


def decoder_layer(x, tensors: dict, config: dict, layer: int, positions) -> np.ndarray:
    """Pre-norm block: `x += attn(norm(x))`, `x += mlp(norm(x))`
    (`src/microinfer/model.py:366-399`)."""
    prefix = f"model.layers.{layer}."
    head_dim = config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]
    eps = config["rms_norm_eps"]
    attn_w = {k[len(prefix) + len("self_attn."):]: v for k, v in tensors.items()
              if k.startswith(prefix + "self_attn.")}
    mlp_w = {k[len(prefix) + len("mlp."):]: v for k, v in tensors.items()
             if k.startswith(prefix + "mlp.")}
    h = rms_norm(x, tensors[prefix + "input_layernorm.weight"], eps)
    x = x + attention(h, attn_w, config["num_attention_heads"], config["num_key_value_heads"],
                      head_dim, config["rope_theta"], positions, layer_window(config, layer))
    h = rms_norm(x, tensors[prefix + "post_attention_layernorm.weight"], eps)
    return x + swiglu_mlp(h, mlp_w)


def hidden_states(config: dict, tensors: dict, ids) -> list[np.ndarray]:
    """The residual stream after the embedding and after every layer, the last
    one after the final norm: the order of the reference's float64 model
    (`tools/conditioning.py:60-82`)."""
    ids = np.asarray(ids)
    positions = np.arange(len(ids))
    x = embed(tensors["model.embed_tokens.weight"], ids)
    states = [x]
    last = config["num_hidden_layers"] - 1
    for layer in range(config["num_hidden_layers"]):
        x = decoder_layer(x, tensors, config, layer, positions)
        states.append(rms_norm(x, tensors["model.norm.weight"], config["rms_norm_eps"])
                      if layer == last else x)
    return states


def cache_contents(config: dict, tensors: dict, ids) -> tuple[np.ndarray, np.ndarray]:
    """What a cache holds after the whole sequence: per layer the rotated keys (with their
    bias, `tools/conditioning.py:70-71`) and the values, each (layers, n, kv_heads,
    head_dim). The reference reads its own cache back the same way
    (`src/microinfer/engine.py:1819-1834`; there the keys are stored without the bias)."""
    ids = np.asarray(ids)
    n = len(ids)
    positions = np.arange(n)
    kv_heads = config["num_key_value_heads"]
    head_dim = config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]
    cos, sin = rope_angles(positions, head_dim, config["rope_theta"])
    x = embed(tensors["model.embed_tokens.weight"], ids)
    keys, values = [], []
    for layer in range(config["num_hidden_layers"]):
        a = f"model.layers.{layer}.self_attn."
        h = rms_norm(x, tensors[f"model.layers.{layer}.input_layernorm.weight"],
                     config["rms_norm_eps"])
        k = linear(h, tensors[a + "k_proj.weight"], tensors[a + "k_proj.bias"])
        v = linear(h, tensors[a + "v_proj.weight"], tensors[a + "v_proj.bias"])
        keys.append(rotate_half(k.reshape(n, kv_heads, head_dim), cos, sin))
        values.append(v.reshape(n, kv_heads, head_dim))
        x = decoder_layer(x, tensors, config, layer, positions)
    return np.stack(keys), np.stack(values)


def lm_head(normed, config: dict, tensors: dict) -> np.ndarray:
    """`logits = y head^T`, the head being the embedding when
    `tie_word_embeddings` (`src/microinfer/model.py:76, 405-413`)."""
    head = (tensors["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False)
            else tensors["lm_head.weight"])
    return normed @ head.T


def forward(config: dict, tensors: dict, ids, rows=None) -> np.ndarray:
    """Logits `(len(ids), vocab)` of one whole sequence
    (`src/microinfer/engine.py:1157-1178`); with `rows`, of those positions only
    (a large vocabulary makes the head the longest part of this slow model)."""
    normed = hidden_states(config, tensors, ids)[-1]
    return lm_head(normed if rows is None else normed[np.asarray(rows)], config, tensors)


# --------------------------------------------------------------------------
# Choosing a token
# --------------------------------------------------------------------------


def greedy(logits: np.ndarray) -> int:
    """The largest logit, the lowest index on a tie, NaN never wins
    (`src/core_kernels/argmax.cu:19-26`)."""
    best, at = -np.inf, len(logits)
    for i, v in enumerate(np.asarray(logits, dtype=np.float64)):
        if v > best:
            best, at = v, i
    return at


_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def _splitmix64(z: np.ndarray) -> np.ndarray:
    z = (z + _GOLDEN).astype(np.uint64)
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)).astype(np.uint64)
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)).astype(np.uint64)
    return z ^ (z >> np.uint64(31))


def gumbel_noise(seed: int, request: int, step: int, vocab: int) -> np.ndarray:
    """The noise of the engine's temperature sampler, which the reference does
    not have (it is greedy only, `src/core_kernels/argmax.cu`): for every
    vocabulary index one uniform number from a counter-based hash of
    (seed, request, step, index), turned into Gumbel noise `-log(-log u)` in
    float32. Written here from the sampler's specification, not from its code."""
    with np.errstate(over="ignore"):
        key = _splitmix64(np.array([seed], dtype=np.uint64)
                          + _GOLDEN * np.uint64(request + 1))
        key = _splitmix64(key ^ (np.uint64(step) * np.uint64(0xD1B54A32D192ED03)))
        z = _splitmix64(key + np.arange(vocab, dtype=np.uint64) * _GOLDEN)
    k = (z >> np.uint64(41)).astype(np.float32)
    u = (k + np.float32(0.5)) * np.float32(2.0 ** -23)
    return -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)


def sample(logits: np.ndarray, temperature: float, seed: int, request: int, step: int) -> int:
    """Greedy at temperature 0; else one draw from `softmax(logits / T)` by the
    Gumbel-max rule: the index that maximises `logits / T + noise`."""
    if temperature == 0.0:
        return greedy(logits)
    scaled = (np.asarray(logits, dtype=np.float32) / np.float32(temperature)
              + gumbel_noise(seed, request, step, len(logits)))
    return greedy(scaled)


def generate(config: dict, tensors: dict, prompt, max_new_tokens: int, *,
             stop_token_ids=(), temperature: float = 0.0, seed: int = 0,
             request: int = 0) -> list[int]:
    """New tokens of one prompt, every step a forward pass over the whole
    sequence so far. Stops after `max_new_tokens` or at a stop token, which is
    kept (`src/microinfer/engine.py:1180-1206, 1244-1253`)."""
    ids = list(prompt)
    out: list[int] = []
    while len(out) < max_new_tokens and not (out and out[-1] in stop_token_ids):
        logits = forward(config, tensors, ids)[-1]
        out.append(sample(logits, temperature, seed, request, len(out)))
        ids.append(out[-1])
    return out

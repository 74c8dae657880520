"""Qwen2 dense decoder: its config.json keys, typed and checked.

The keys and their meaning follow the reference's `ModelConfig`
(`src/microinfer/config.py:24-46, 64-88`) and its committed model cards
(`src/microinfer/model_cards/qwen2.5-1.5b-instruct.json`). The reference
requires thirteen keys and derives `head_dim = hidden_size //
num_attention_heads` (`config.py:48-52`); here `head_dim` may also be given,
and the window keys of the card (`use_sliding_window`, `sliding_window`,
`max_window_layers`), which the reference never reads, choose a windowed
attention for the layers from `max_window_layers` on.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Optional

from .registry import register_architecture
from .specs import (AttentionSpec, BlockSpec, ConfigError, GatedMLPSpec, LayerCall, ModelSpec,
                    NormSpec, RotarySpec)

_REQUIRED = {
    "num_hidden_layers": int, "hidden_size": int, "num_attention_heads": int,
    "num_key_value_heads": int, "intermediate_size": int, "vocab_size": int,
    "max_position_embeddings": int, "rope_theta": (int, float), "rms_norm_eps": float,
}


@dataclass(frozen=True)
class Qwen2Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    hidden_act: str
    torch_dtype: str
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    eos_token_id: tuple
    bos_token_id: Optional[int]
    initializer_range: float

    architecture = "Qwen2ForCausalLM"

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2Config":
        problems = []
        for key, kind in _REQUIRED.items():
            if key not in raw:
                problems.append(f"{key}: missing")
            elif isinstance(raw[key], bool) or not isinstance(raw[key], kind):
                problems.append(f"{key}: expected a number, config.json has {raw[key]!r}")
        if problems:
            raise ConfigError("config.json cannot describe a Qwen2 model:\n    "
                              + "\n    ".join(problems))

        def positive(key):
            if raw[key] <= 0:
                problems.append(f"{key}: must be positive, config.json has {raw[key]!r}")

        for key in _REQUIRED:
            positive(key)
        heads, kv_heads, hidden = (raw["num_attention_heads"], raw["num_key_value_heads"],
                                   raw["hidden_size"])
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if heads > 0 and hidden % heads:
                problems.append(f"hidden_size {hidden} is not a multiple of "
                                f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // max(heads, 1)
        elif isinstance(head_dim, bool) or not isinstance(head_dim, int) or head_dim <= 0:
            problems.append(f"head_dim: expected a positive integer, config.json has {head_dim!r}")
            head_dim = 0
        if head_dim % 2:
            problems.append(f"head_dim {head_dim} is odd; rotary pairs need an even size")
        if kv_heads > 0 and heads % kv_heads:
            problems.append(f"num_attention_heads {heads} is not a multiple of "
                            f"num_key_value_heads {kv_heads}")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            problems.append(f"hidden_act {act!r}: only 'silu' is built")
        if raw.get("rope_scaling") not in (None, {}):
            problems.append(f"rope_scaling {raw['rope_scaling']!r}: scaled rotary positions "
                            "are not built")
        use_window = bool(raw.get("use_sliding_window", False))
        window = raw.get("sliding_window")
        if use_window and (not isinstance(window, int) or isinstance(window, bool) or window <= 0):
            problems.append("use_sliding_window is on but sliding_window is "
                            f"{window!r}, not a positive integer")
        max_window_layers = raw.get("max_window_layers", raw["num_hidden_layers"])
        if isinstance(max_window_layers, bool) or not isinstance(max_window_layers, int) \
                or max_window_layers < 0:
            problems.append(f"max_window_layers {max_window_layers!r}: expected an integer >= 0")
            max_window_layers = raw["num_hidden_layers"]
        dtype = raw.get("torch_dtype", raw.get("dtype", "bfloat16"))
        if dtype not in ("bfloat16", "float32", "float16"):
            problems.append(f"torch_dtype {dtype!r}: expected bfloat16, float16 or float32")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)
        for e in eos:
            if isinstance(e, bool) or not isinstance(e, int):
                problems.append(f"eos_token_id {raw.get('eos_token_id')!r}: expected integers")
                eos = ()
                break
        if problems:
            raise ConfigError("config.json cannot describe a Qwen2 model:\n    "
                              + "\n    ".join(problems))
        return cls(
            num_hidden_layers=raw["num_hidden_layers"], hidden_size=hidden,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            intermediate_size=raw["intermediate_size"], vocab_size=raw["vocab_size"],
            max_position_embeddings=raw["max_position_embeddings"],
            rope_theta=float(raw["rope_theta"]), rms_norm_eps=float(raw["rms_norm_eps"]),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            hidden_act=act, torch_dtype=dtype, use_sliding_window=use_window,
            sliding_window=window if use_window else None,
            max_window_layers=max_window_layers, eos_token_id=eos,
            bos_token_id=raw.get("bos_token_id"),
            initializer_range=float(raw.get("initializer_range", 0.02)))

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        raw = asdict(self)
        raw["architectures"] = [self.architecture]
        raw["model_type"] = "qwen2"
        raw["eos_token_id"] = (list(self.eos_token_id) if len(self.eos_token_id) != 1
                               else self.eos_token_id[0]) if self.eos_token_id else None
        return raw

    def window_of(self, layer: int) -> Optional[int]:
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    @property
    def kv_bytes_per_token(self) -> int:
        """Keys and values of one token over all layers at two bytes an element
        (`src/microinfer/config.py:54-62`)."""
        return 2 * self.num_hidden_layers * self.num_key_value_heads * self.head_dim * 2

    def model_spec(self) -> ModelSpec:
        rotary = RotarySpec(head_dim=self.head_dim, rotary_dim=self.head_dim,
                            theta=self.rope_theta, max_positions=self.max_position_embeddings)
        norm = NormSpec(size=self.hidden_size, eps=self.rms_norm_eps)
        mlp = GatedMLPSpec(hidden=self.hidden_size, intermediate=self.intermediate_size,
                           activation=self.hidden_act)
        blocks = []
        for layer in range(self.num_hidden_layers):
            attention = AttentionSpec(
                hidden=self.hidden_size, heads=self.num_attention_heads,
                kv_heads=self.num_key_value_heads, head_dim=self.head_dim, qkv_bias=True,
                out_bias=False, scale=1.0 / math.sqrt(self.head_dim),
                window=self.window_of(layer), position=rotary)
            blocks.append(BlockSpec(prefix=f"model.layers.{layer}.", mixer=attention,
                                    mixer_norm=norm, ffn=mlp, ffn_norm=norm))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden=self.hidden_size,
            blocks=tuple(blocks),
            run_order=tuple(LayerCall(block=i, cache=i) for i in range(self.num_hidden_layers)),
            final_norm=norm, tie_head=self.tie_word_embeddings,
            max_positions=self.max_position_embeddings, stop_token_ids=self.eos_token_id,
            stored_dtype=self.torch_dtype, init_std=self.initializer_range,
            # exporters of this architecture have written the rotary table's frequencies
            ignore_tensors=("*.rotary_emb.inv_freq",))


register_architecture(Qwen2Config.architecture, Qwen2Config)

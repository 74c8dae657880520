"""What a model is made of, as plain data.

A configuration class (one per architecture) reads that architecture's own
config.json keys and turns them into a `ModelSpec`: a list of block
descriptions, each naming its mixer, feed-forward, norms and position encoding
with every size and constant as a field, plus the order in which the blocks
run. The parts are built from these descriptions alone; no part ever sees a
config.json or knows which architecture it belongs to.

Every spec has a `kind`: the name under which a part class is registered in
`parts.registry`. A new kind of mixer, feed-forward, norm or position encoding
is a new spec dataclass with a new `kind` and a registered part class; nothing
here needs to change for it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


class ConfigError(ValueError):
    """A config.json this library cannot run; the message names every problem."""


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    kind: str = "rms_norm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotate-half rotary position encoding of the first `rotary_dim` of each head."""
    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rotary_half"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal self-attention over cached keys and values.

    `window` None means every earlier key is seen; a number w means the last w
    keys, the query's own included.
    """
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    qkv_bias: bool
    out_bias: bool
    scale: float
    window: Optional[int]
    position: Optional[RotarySpec]
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: `down(act(gate(x)) * up(x))`."""
    hidden: int
    intermediate: int
    activation: str
    bias: bool = False
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: how a mixer and a feed-forward are arranged around the residual.

    `prefix` is where the block's tensors sit in the checkpoint
    ("model.layers.3."); the parts append their own names to it.
    """
    prefix: str
    mixer: object
    mixer_norm: NormSpec
    ffn: object
    ffn_norm: NormSpec
    mixer_name: str = "self_attn"
    ffn_name: str = "mlp"
    mixer_norm_name: str = "input_layernorm"
    ffn_norm_name: str = "post_attention_layernorm"
    kind: str = "pre_norm"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run block `block` with cache entry `cache`.

    A cache entry belongs to the first call that names it, which writes it;
    later calls with the same entry only read it (a layer that reads another
    layer's cache). A block may appear in several calls (a layer run twice);
    each such call needs a cache entry of its own unless it shares one on
    purpose.
    """
    block: int
    cache: int


@dataclass(frozen=True)
class ModelSpec:
    """`embed_scale` multiplies the embedding's rows as they enter the residual stream;
    `logit_scale` multiplies the logits and `logit_softcap` c then bends them to
    `c * tanh(logits / c)` (None: neither); `head_bias_name` names a bias [vocab] of the
    output head. `ignore_tensors`: shell-style patterns of tensor names that a checkpoint
    of this architecture may hold without any part reading them (buffers that exporters
    write, such as a rotary table's `inv_freq`); anything else unexpected is an error."""
    architecture: str
    vocab_size: int
    hidden: int
    blocks: tuple
    run_order: tuple
    final_norm: NormSpec
    tie_head: bool
    max_positions: int
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    stop_token_ids: tuple = ()
    stored_dtype: str = "bfloat16"
    init_std: float = 0.02
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    head_bias_name: Optional[str] = None
    ignore_tensors: tuple = ()

    def cache_entries(self) -> int:
        return 1 + max((c.cache for c in self.run_order), default=-1)

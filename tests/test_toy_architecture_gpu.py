"""A toy architecture defined here, outside the package: a mixer with running
state of its own (fixed size per sequence), used beside the package's attention
in one model, with a layer that runs twice and a layer that reads another
layer's cache. It is registered, written as a random checkpoint, loaded, and
stepped whole, token by token and in unequal batches, without any change to the
package's files, and compared with a plain NumPy version written below."""

import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_model as plain
import semantic_aware_adaptive_kv_cache_precision_b200 as sakv
from semantic_aware_adaptive_kv_cache_precision_b200.cache import StateNeed
from semantic_aware_adaptive_kv_cache_precision_b200.config import (AttentionSpec, BlockSpec,
                                                                     GatedMLPSpec, LayerCall,
                                                                     ModelSpec, NormSpec,
                                                                     RotarySpec)
from semantic_aware_adaptive_kv_cache_precision_b200.parts import Part, register_part
from semantic_aware_adaptive_kv_cache_precision_b200.weights import TensorDecl
from helpers import assert_same_logits

pytestmark = pytest.mark.gpu


# ---- the toy mixer: s_t = decay * s_{t-1} + W_in h_t ;  out_t = W_out s_t -----------------

@dataclass(frozen=True)
class RunningStateSpec:
    hidden: int
    state: int
    decay: float
    kind: str = "toy_running_state"


class RunningStateMixer(Part):
    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(self.prefix + "in_proj.weight", (s.state, s.hidden)),
                TensorDecl(self.prefix + "out_proj.weight", (s.hidden, s.state))]

    def bind(self, arena):
        self.w_in = arena.view(self.prefix + "in_proj.weight")
        self.w_out = arena.view(self.prefix + "out_proj.weight")

    def cache_need(self):
        return StateNeed((self.spec.state,), "float32")

    def forward(self, h, step, view, residual, write_cache=True):
        u = h.float() @ self.w_in.float().t()
        out = torch.empty_like(u)
        at = 0
        for slot, count in zip(step.host_slots, step.new_counts):
            s = view.state[slot].clone()
            for t in range(at, at + count):
                s = self.spec.decay * s + u[t]
                out[t] = s
            view.state[slot] = s
            at += count
        residual += out @ self.w_out.float().t()


register_part("toy_running_state", RunningStateMixer)


# ---- the toy architecture -------------------------------------------------------------------

@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int = 48
    state_size: int = 20
    decay: float = 0.8
    num_attention_heads: int = 3
    num_key_value_heads: int = 1
    intermediate_size: int = 72
    vocab_size: int = 211
    rms_norm_eps: float = 1e-5
    rope_theta: float = 3000.0
    max_position_embeddings: int = 256

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: raw[k] for k in cls.__dataclass_fields__ if k in raw})

    def to_dict(self):
        return {**self.__dict__, "architectures": ["ToyMixedForTests"]}

    def model_spec(self):
        h, d = self.hidden_size, self.hidden_size // self.num_attention_heads
        norm = NormSpec(h, self.rms_norm_eps)
        mlp = GatedMLPSpec(h, self.intermediate_size, "silu")
        rotary = RotarySpec(d, d, self.rope_theta, self.max_position_embeddings)
        attn = AttentionSpec(hidden=h, heads=self.num_attention_heads,
                             kv_heads=self.num_key_value_heads, head_dim=d, qkv_bias=True,
                             out_bias=False, scale=d ** -0.5, window=None, position=rotary)
        blocks = (BlockSpec("model.layers.0.", RunningStateSpec(h, self.state_size, self.decay),
                            norm, mlp, norm, mixer_name="mixer"),
                  BlockSpec("model.layers.1.", attn, norm, mlp, norm),
                  BlockSpec("model.layers.2.", attn, norm, mlp, norm))
        # block 0 runs twice (two states); block 2 reads the cache that block 1 wrote
        order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 1))
        return ModelSpec(architecture="ToyMixedForTests", vocab_size=self.vocab_size, hidden=h,
                         blocks=blocks, run_order=order, final_norm=norm, tie_head=True,
                         max_positions=self.max_position_embeddings, stored_dtype="float32")


sakv.register_architecture("ToyMixedForTests", ToyConfig)


# ---- its plain version ------------------------------------------------------------------------

def plain_toy(config: ToyConfig, t: dict, ids) -> np.ndarray:
    n = len(ids)
    heads, kvh = config.num_attention_heads, config.num_key_value_heads
    d = config.hidden_size // heads
    cos, sin = plain.rope_angles(np.arange(n), d, config.rope_theta)
    eps = config.rms_norm_eps

    def mlp(x, p):
        w = {k[len(p + "mlp."):]: v for k, v in t.items() if k.startswith(p + "mlp.")}
        return x + plain.swiglu_mlp(plain.rms_norm(x, t[p + "post_attention_layernorm.weight"], eps), w)

    def state_layer(x):
        p = "model.layers.0."
        h = plain.rms_norm(x, t[p + "input_layernorm.weight"], eps)
        u = h @ t[p + "mixer.in_proj.weight"].T
        s, out = np.zeros(config.state_size), np.empty_like(u)
        for i in range(n):
            s = config.decay * s + u[i]
            out[i] = s
        return mlp(x + out @ t[p + "mixer.out_proj.weight"].T, p)

    def attn_layer(x, p, kv=None):
        h = plain.rms_norm(x, t[p + "input_layernorm.weight"], eps)
        a = p + "self_attn."
        q = plain.rotate_half(plain.linear(h, t[a + "q_proj.weight"], t[a + "q_proj.bias"])
                              .reshape(n, heads, d), cos, sin)
        if kv is None:
            k = plain.rotate_half(plain.linear(h, t[a + "k_proj.weight"], t[a + "k_proj.bias"])
                                  .reshape(n, kvh, d), cos, sin)
            v = plain.linear(h, t[a + "v_proj.weight"], t[a + "v_proj.bias"]).reshape(n, kvh, d)
            kv = (k, v)
        k, v = kv
        out = np.empty((n, heads, d))
        for hd in range(heads):
            g = hd // (heads // kvh)
            s = np.where(plain.causal_mask(n), q[:, hd] @ k[:, g].T / np.sqrt(d), -np.inf)
            out[:, hd] = plain.softmax(s) @ v[:, g]
        x = x + out.reshape(n, -1) @ t[a + "o_proj.weight"].T
        return mlp(x, p), kv

    x = plain.embed(t["model.embed_tokens.weight"], ids)
    x = state_layer(x)
    x, kv = attn_layer(x, "model.layers.1.")
    x = state_layer(x)
    x, _ = attn_layer(x, "model.layers.2.", kv)
    return plain.rms_norm(x, t["model.norm.weight"], eps) @ t["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_registers_builds_and_steps(dtype, tmp_path):
    config = ToyConfig()
    folder = sakv.write_random_model(tmp_path / "toy", config, seed=3)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyMixedForTests"]
    engine = sakv.Engine(folder, dtype=dtype, max_tokens=1024, poison_freed=True).load_weights()
    needs = engine.model.cache_needs()
    assert [type(n).__name__ for n in needs] == ["StateNeed", "KVNeed", "StateNeed"]
    _, tensors = plain.read_model_folder(folder)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, config.vocab_size, n) for n in (70, 9, 131)]
    want = [plain_toy(config, tensors, p) for p in prompts]
    tol = 2e-5 if dtype == "float32" else 0.06
    whole = [engine.forward(p) for p in prompts]
    for g, w in zip(whole, want):
        scale = np.abs(w).max() if dtype == "float32" else w.std()
        assert np.abs(g - w).max() <= tol * scale
    # token by token: the running state is carried in the slot
    (slot,) = engine.open(1)
    rows = [engine.step([slot], [prompts[1][i:i + 1]]).cpu().numpy() for i in range(9)]
    engine.close([slot])
    assert np.abs(np.concatenate(rows) - whole[1]).max() <= tol * np.abs(whole[1]).max()
    # an unequal batch, three times in a row, so that slots (and their state) are used again:
    # the same slots, then other slots for a batch of the same shape (a captured step that
    # kept the first batch's slot numbers would update the wrong sequences' state), then the
    # first ones in another order
    for round_ in range(3):
        if round_ == 1:
            spare, *slots = engine.open(4)
            engine.close([spare])
        else:
            slots = engine.open(3)[::-1] if round_ == 2 else engine.open(3)
        heads = [len(p) - 4 for p in prompts]
        out = engine.step(slots, [p[:h] for p, h in zip(prompts, heads)],
                          [list(range(h)) for h in heads]).cpu().numpy()
        rows = [[out[sum(heads[:i]):sum(heads[:i + 1])]] for i in range(3)]
        for t in range(4):
            out = engine.step(slots, [p[h + t:h + t + 1] for p, h in zip(prompts, heads)])
            for i in range(3):
                rows[i].append(out[i:i + 1].cpu().numpy())
        engine.close(slots)
        for i in range(3):
            got = np.concatenate(rows[i])
            scale = np.abs(want[i]).max() if dtype == "float32" else want[i].std()
            assert np.abs(got - want[i]).max() <= tol * scale, f"round {round_} request {i}"
    engine.cache.check()
    out = engine.generate([p.tolist() for p in prompts[:2]], 5, stop_at_eos=False)
    assert [len(o) for o in out] == [5, 5]


# ---- a second toy: a routed feed-forward and another position encoding -----------------------
# Attention with a learned table of position vectors added to queries and keys (instead of a
# rotation), and a feed-forward of small experts with top-2 routing. Both are defined here,
# registered from here, and use the package only through its part interfaces.

@dataclass(frozen=True)
class AddedPositionSpec:
    head_dim: int
    max_positions: int
    kind: str = "toy_added_position"


class AddedPosition(Part):
    """q += P[pos], k += P[pos] with a learned table P [positions, head_dim]."""

    def tensor_decls(self):
        return [TensorDecl(self.prefix + "position_table", (self.spec.max_positions,
                                                            self.spec.head_dim))]

    def bind(self, arena):
        self.table = arena.view(self.prefix + "position_table")

    def rotate_store(self, qkv, step, view, heads, kv_heads, head_dim, write_cache=True):
        from semantic_aware_adaptive_kv_cache_precision_b200 import ops
        rows = self.table[step.positions.long()].to(qkv.dtype)             # [T, d]
        qk = qkv[:, :(heads + kv_heads) * head_dim].view(qkv.shape[0], heads + kv_heads, head_dim)
        qk += rows[:, None, :]
        ops.rope_store(qkv, step.positions, step.token_seq, view.block_table, None, None,
                       view.keys, view.values, heads, kv_heads, head_dim, write_cache)


register_part("toy_added_position", AddedPosition)


@dataclass(frozen=True)
class RoutedSpec:
    hidden: int
    inner: int
    experts: int
    top: int
    kind: str = "toy_routed_ffn"


class RoutedFFN(Part):
    """residual += sum over the top experts e of p_e * W2_e silu(W1_e h); the router's
    logits and softmax are fp32."""

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        decls = [TensorDecl(p + "router.weight", (s.experts, s.hidden))]
        for e in range(s.experts):
            decls += [TensorDecl(f"{p}experts.{e}.w1", (s.inner, s.hidden)),
                      TensorDecl(f"{p}experts.{e}.w2", (s.hidden, s.inner))]
        return decls

    def bind(self, arena):
        p = self.prefix
        self.router = arena.view(p + "router.weight")
        self.w1 = [arena.view(f"{p}experts.{e}.w1") for e in range(self.spec.experts)]
        self.w2 = [arena.view(f"{p}experts.{e}.w2") for e in range(self.spec.experts)]

    def forward(self, h, step, residual):
        from semantic_aware_adaptive_kv_cache_precision_b200 import ops
        logits = h.float() @ self.router.float().t()
        top_v, top_i = logits.topk(self.spec.top, dim=-1)
        weight = torch.softmax(top_v, dim=-1)
        for e in range(self.spec.experts):
            rows, which = (top_i == e).nonzero(as_tuple=True)
            if rows.numel() == 0:
                continue
            x = h[rows].contiguous()
            inner = ops.linear(x, self.w1[e], out_dtype=torch.float32)
            act = (inner / (1 + torch.exp(-inner))).to(h.dtype)
            y = ops.linear(act, self.w2[e], out_dtype=torch.float32)
            residual.index_add_(0, rows, y * weight[rows, which][:, None])


register_part("toy_routed_ffn", RoutedFFN)


@dataclass(frozen=True)
class RoutedConfig:
    hidden_size: int = 64
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    inner_size: int = 40
    num_experts: int = 5
    top_k: int = 2
    dense_size: int = 96
    vocab_size: int = 150
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 320

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: raw[k] for k in cls.__dataclass_fields__ if k in raw})

    def to_dict(self):
        return {**self.__dict__, "architectures": ["ToyRoutedForTests"]}

    def model_spec(self):
        h, d = self.hidden_size, self.hidden_size // self.num_attention_heads
        norm = NormSpec(h, self.rms_norm_eps)
        attn = AttentionSpec(hidden=h, heads=self.num_attention_heads,
                             kv_heads=self.num_key_value_heads, head_dim=d, qkv_bias=False,
                             out_bias=True, scale=d ** -0.5, window=None,
                             position=AddedPositionSpec(d, self.max_position_embeddings))
        routed = RoutedSpec(h, self.inner_size, self.num_experts, self.top_k)
        dense = GatedMLPSpec(h, self.dense_size, "silu")
        # layer 0: routed feed-forward, layer 1: dense, layer 2: routed
        blocks = tuple(BlockSpec(f"model.layers.{i}.", attn, norm, ffn, norm)
                       for i, ffn in enumerate((routed, dense, routed)))
        return ModelSpec(architecture="ToyRoutedForTests", vocab_size=self.vocab_size, hidden=h,
                         blocks=blocks, run_order=tuple(LayerCall(i, i) for i in range(3)),
                         final_norm=norm, tie_head=False,
                         max_positions=self.max_position_embeddings, stored_dtype="float32")


sakv.register_architecture("ToyRoutedForTests", RoutedConfig)


def plain_routed(config: RoutedConfig, t: dict, ids) -> np.ndarray:
    n = len(ids)
    heads, kvh = config.num_attention_heads, config.num_key_value_heads
    d = config.hidden_size // heads
    eps = config.rms_norm_eps
    x = plain.embed(t["model.embed_tokens.weight"], ids)
    for i in range(3):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        h = plain.rms_norm(x, t[p + "input_layernorm.weight"], eps)
        table = t[a + "position_table"][:n]
        q = plain.linear(h, t[a + "q_proj.weight"]).reshape(n, heads, d) + table[:, None, :]
        k = plain.linear(h, t[a + "k_proj.weight"]).reshape(n, kvh, d) + table[:, None, :]
        v = plain.linear(h, t[a + "v_proj.weight"]).reshape(n, kvh, d)
        out = np.empty((n, heads, d))
        for hd in range(heads):
            g = hd // (heads // kvh)
            s = np.where(plain.causal_mask(n), q[:, hd] @ k[:, g].T / np.sqrt(d), -np.inf)
            out[:, hd] = plain.softmax(s) @ v[:, g]
        x = x + plain.linear(out.reshape(n, -1), t[a + "o_proj.weight"], t[a + "o_proj.bias"])
        h = plain.rms_norm(x, t[p + "post_attention_layernorm.weight"], eps)
        if i == 1:
            w = {k_[len(p + "mlp."):]: v_ for k_, v_ in t.items() if k_.startswith(p + "mlp.")}
            x = x + plain.swiglu_mlp(h, w)
            continue
        logits = h @ t[p + "mlp.router.weight"].T
        y = np.zeros_like(x)
        for row in range(n):
            top = np.argsort(-logits[row], kind="stable")[:config.top_k]
            pw = plain.softmax(logits[row, top][None, :])[0]
            for e, pe in zip(top, pw):
                inner = h[row] @ t[f"{p}mlp.experts.{e}.w1"].T
                y[row] += pe * ((inner / (1 + np.exp(-inner))) @ t[f"{p}mlp.experts.{e}.w2"].T)
        x = x + y
    return plain.rms_norm(x, t["model.norm.weight"], eps) @ t["lm_head.weight"].T


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    config = RoutedConfig()
    folder = sakv.write_random_model(tmp_path / "routed", config, seed=7)
    engine = sakv.Engine(folder, dtype="float32", max_tokens=1024).load_weights()
    _, tensors = plain.read_model_folder(folder)
    # make the routing matter: spread the router's logits
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, config.vocab_size, n) for n in (40, 5, 90)]
    want = [plain_routed(config, tensors, p) for p in prompts]
    for p, w in zip(prompts, want):
        got = engine.forward(p)
        assert np.abs(got - w).max() <= 5e-5 * np.abs(w).max()
    slots = engine.open(3)
    heads = [len(p) - 3 for p in prompts]
    out = engine.step(slots, [p[:h] for p, h in zip(prompts, heads)],
                      [list(range(h)) for h in heads]).cpu().numpy()
    rows = [[out[sum(heads[:i]):sum(heads[:i + 1])]] for i in range(3)]
    for t_ in range(3):
        step_out = engine.step(slots, [p[h + t_:h + t_ + 1] for p, h in zip(prompts, heads)])
        for i in range(3):
            rows[i].append(step_out[i:i + 1].cpu().numpy())
    engine.close(slots)
    for i in range(3):
        assert np.abs(np.concatenate(rows[i]) - want[i]).max() <= 5e-5 * np.abs(want[i]).max()


# ---- a third toy: keys and values of different widths, and the model-level hooks --------------
# A mixer that caches keys of width 8 and values of width 20 for each position (its cache
# need says so; the cache gives it storage of that shape), beside the package's attention in
# one model whose spec scales the embedding, scales and soft-caps the logits, has a bias on
# its output head, and lets a checkpoint carry a buffer that no part reads.

@dataclass(frozen=True)
class NarrowKeySpec:
    hidden: int
    key_dim: int
    value_dim: int
    kind: str = "toy_narrow_keys"


class NarrowKeyMixer(Part):
    """out_t = W_o sum_{j <= t} softmax_j(q_t . k_j / sqrt(dk)) v_j with k of width dk and v
    of width dv: one KV head, no position encoding."""

    graph_safe = False      # its launches depend on the sequences' lengths on the host

    def tensor_decls(self):
        s, p = self.spec, self.prefix
        return [TensorDecl(p + "q.weight", (s.key_dim, s.hidden)),
                TensorDecl(p + "k.weight", (s.key_dim, s.hidden)),
                TensorDecl(p + "v.weight", (s.value_dim, s.hidden)),
                TensorDecl(p + "o.weight", (s.hidden, s.value_dim))]

    def bind(self, arena):
        p = self.prefix
        self.wq, self.wk, self.wv, self.wo = (arena.view(p + n + ".weight").float()
                                              for n in "qkvo")

    def cache_need(self):
        from semantic_aware_adaptive_kv_cache_precision_b200.cache import KVNeed
        return KVNeed(1, self.spec.key_dim, value_dim=self.spec.value_dim, dtype="float32")

    def forward(self, h, step, view, residual, write_cache=True):
        h = h.float()
        q, k, v = h @ self.wq.t(), h @ self.wk.t(), h @ self.wv.t()
        assert view.keys.shape[1:] == (1, 64, self.spec.key_dim)
        assert view.values.shape[1:] == (1, 64, self.spec.value_dim)
        seq, pos = step.token_seq.long(), step.positions.long()
        block = view.block_table[seq, pos // 64].long()
        if write_cache:
            view.keys[block, 0, pos % 64] = k
            view.values[block, 0, pos % 64] = v
        out = torch.empty_like(v)
        at = 0
        for i, (start, count) in enumerate(zip(step.starts, step.new_counts)):
            blocks = view.block_table[i, :-(-(start + count) // 64)].long()
            keys = view.keys[blocks, 0].reshape(-1, self.spec.key_dim)[:start + count]
            values = view.values[blocks, 0].reshape(-1, self.spec.value_dim)[:start + count]
            scores = q[at:at + count] @ keys.t() / self.spec.key_dim ** 0.5
            seen = torch.arange(start + count, device=h.device)[None, :] <= \
                (start + torch.arange(count, device=h.device))[:, None]
            out[at:at + count] = torch.softmax(scores.masked_fill(~seen, float("-inf")), -1) @ values
            at += count
        residual += out @ self.wo.t()


register_part("toy_narrow_keys", NarrowKeyMixer)


@dataclass(frozen=True)
class HookedConfig:
    hidden_size: int = 64
    key_dim: int = 8
    value_dim: int = 20
    num_attention_heads: int = 2
    intermediate_size: int = 56
    vocab_size: int = 97
    rms_norm_eps: float = 1e-5
    max_position_embeddings: int = 192
    embed_scale: float = 2.0
    logit_scale: float = 0.5
    logit_softcap: float = 2.0

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: raw[k] for k in cls.__dataclass_fields__ if k in raw})

    def to_dict(self):
        return {**self.__dict__, "architectures": ["ToyHookedForTests"]}

    def model_spec(self):
        h, d = self.hidden_size, self.hidden_size // self.num_attention_heads
        norm = NormSpec(h, self.rms_norm_eps)
        mlp = GatedMLPSpec(h, self.intermediate_size, "silu")
        attn = AttentionSpec(hidden=h, heads=self.num_attention_heads, kv_heads=1, head_dim=d,
                             qkv_bias=True, out_bias=False, scale=d ** -0.5, window=None,
                             position=RotarySpec(d, d, 1e4, self.max_position_embeddings))
        blocks = (BlockSpec("model.layers.0.", NarrowKeySpec(h, self.key_dim, self.value_dim),
                            norm, mlp, norm, mixer_name="mixer"),
                  BlockSpec("model.layers.1.", attn, norm, mlp, norm))
        return ModelSpec(architecture="ToyHookedForTests", vocab_size=self.vocab_size, hidden=h,
                         blocks=blocks, run_order=(LayerCall(0, 0), LayerCall(1, 1)),
                         final_norm=norm, tie_head=False,
                         max_positions=self.max_position_embeddings, stored_dtype="float32",
                         init_std=0.1, embed_scale=self.embed_scale,
                         logit_scale=self.logit_scale, logit_softcap=self.logit_softcap,
                         head_bias_name="lm_head.bias", ignore_tensors=("*.unused_buffer",))


sakv.register_architecture("ToyHookedForTests", HookedConfig)


def plain_hooked(config: HookedConfig, t: dict, ids) -> np.ndarray:
    n = len(ids)
    heads = config.num_attention_heads
    d = config.hidden_size // heads
    eps = config.rms_norm_eps
    x = plain.embed(t["model.embed_tokens.weight"], ids) * config.embed_scale
    p = "model.layers.0."
    h = plain.rms_norm(x, t[p + "input_layernorm.weight"], eps)
    q, k, v = (h @ t[p + f"mixer.{n_}.weight"].T for n_ in "qkv")
    s = np.where(plain.causal_mask(n), q @ k.T / np.sqrt(config.key_dim), -np.inf)
    x = x + (plain.softmax(s) @ v) @ t[p + "mixer.o.weight"].T
    w = {k_[len(p + "mlp."):]: v_ for k_, v_ in t.items() if k_.startswith(p + "mlp.")}
    x = x + plain.swiglu_mlp(plain.rms_norm(x, t[p + "post_attention_layernorm.weight"], eps), w)
    raw = {"num_hidden_layers": 2, "hidden_size": config.hidden_size, "num_attention_heads": heads,
           "num_key_value_heads": 1, "rope_theta": 1e4, "rms_norm_eps": eps}
    x = plain.decoder_layer(x, t, raw, 1, np.arange(n))
    logits = plain.rms_norm(x, t["model.norm.weight"], eps) @ t["lm_head.weight"].T
    logits = (logits + t["lm_head.bias"]) * config.logit_scale
    return config.logit_softcap * np.tanh(logits / config.logit_softcap)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_and_values_of_different_widths_and_the_models_hooks(dtype, tmp_path):
    from semantic_aware_adaptive_kv_cache_precision_b200.weights import (SafetensorsFile,
                                                                          write_safetensors)
    config = HookedConfig()
    folder = sakv.write_random_model(tmp_path / "hooked", config, seed=11)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.infos}
    del f
    assert tensors["lm_head.bias"].abs().sum() == 0           # written as zeros: make it matter
    tensors["lm_head.bias"] = torch.linspace(-2, 2, config.vocab_size)
    tensors["model.layers.0.mixer.unused_buffer"] = torch.ones(3)   # let pass by the spec
    write_safetensors(folder / "model.safetensors", tensors)
    engine = sakv.Engine(folder, dtype=dtype, max_tokens=1024, poison_freed=True).load_weights()
    needs = engine.model.cache_needs()
    assert needs[0].head_dim == 8 and needs[0].value_dim == 20 and needs[1].value_dim is None
    _, plain_tensors = plain.read_model_folder(folder)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, config.vocab_size, n) for n in (70, 3, 130)]
    want = [plain_hooked(config, plain_tensors, p) for p in prompts]
    assert max(np.abs(w).max() for w in want) > 1.5           # the cap (2.0) bends something
    tol = 2e-5 if dtype == "float32" else 0.06
    for p, w in zip(prompts, want):
        scale = np.abs(w).max() if dtype == "float32" else w.std()
        assert np.abs(engine.forward(p) - w).max() <= tol * scale
    group = engine.cache.groups[engine.cache.entry_group[0][0]]
    assert group.keys.shape[-1] == 8 and group.values.shape[-1] == 20
    assert group.keys.dtype == torch.float32
    # an unequal batch with the last tokens one by one, twice, so that blocks are used again
    for _ in range(2):
        slots = engine.open(3)
        heads = [len(p) - 2 for p in prompts]
        out = engine.step(slots, [p[:h] for p, h in zip(prompts, heads)],
                          [list(range(h)) for h in heads]).cpu().numpy()
        rows = [[out[sum(heads[:i]):sum(heads[:i + 1])]] for i in range(3)]
        for t_ in range(2):
            step_out = engine.step(slots, [p[h + t_:h + t_ + 1] for p, h in zip(prompts, heads)])
            for i in range(3):
                rows[i].append(step_out[i:i + 1].cpu().numpy())
        engine.close(slots)
        for i in range(3):
            scale = np.abs(want[i]).max() if dtype == "float32" else want[i].std()
            assert np.abs(np.concatenate(rows[i]) - want[i]).max() <= tol * scale, f"request {i}"
    engine.cache.check()
    assert engine.graph_failure is None and not engine.model.graph_safe

"""Each part alone: built from its spec and handed tensors, run on the device, and
compared with the plain function of the same part. Sizes differ from the tiny
models'."""

import numpy as np
import pytest
import torch

import plain_model as plain
from semantic_aware_adaptive_kv_cache_precision_b200.cache import KVNeed, SequenceCache
from semantic_aware_adaptive_kv_cache_precision_b200.config import (AttentionSpec, BlockSpec,
                                                                     GatedMLPSpec, NormSpec,
                                                                     RotarySpec)
from semantic_aware_adaptive_kv_cache_precision_b200.engine.step import StepStager
from semantic_aware_adaptive_kv_cache_precision_b200.parts import build_part
from semantic_aware_adaptive_kv_cache_precision_b200.weights import WeightArena

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bind(part, mode, seed=0, scale=0.05):
    """Random tensors for every declaration of `part`; returns them as float64."""
    rng = np.random.default_rng(seed)
    decls = part.tensor_decls()
    dtype = torch.float32 if mode == "float32" else torch.bfloat16
    arena = WeightArena(decls, {d.name: dtype for d in decls}, DEV)
    values = {}
    for d in decls:
        v = rng.standard_normal(d.shape) * scale + (1.0 if d.init == "ones_normal" else 0.0)
        t = torch.as_tensor(v).to(dtype)
        arena.view(d.name).copy_(t)
        values[d.name] = t.double().numpy()
    part.bind(arena)
    return values


def step_for(cache, stager, slots, token_lists):
    starts = [int(cache.lengths[s]) for s in slots]
    ends = [a + len(t) for a, t in zip(starts, token_lists)]
    cache.reserve(slots, ends)
    ctx = stager.build(slots, token_lists, starts, [], cache.tables_for(slots))
    return ctx, ends


# relative to the largest value of the expected output: a few fp32 roundings, or a few
# bf16 roundings (2^-9 each) on the way
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def close(got, want, mode, factor=1.0, err_msg=""):
    np.testing.assert_allclose(got, want, rtol=0, atol=factor * TOL[mode] * np.abs(want).max(),
                               err_msg=err_msg)


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_norm_part(mode):
    part = build_part(NormSpec(size=136, eps=2e-4), "some.norm", mode)
    values = bind(part, mode, scale=0.3)
    x = torch.randn(5, 136, device=DEV) * 2
    got = part.forward(x)
    assert got.dtype == part.act_dtype
    want = plain.rms_norm(x.double().cpu().numpy(), values["some.norm.weight"], 2e-4)
    close(got.double().cpu().numpy(), want, mode)


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 40])
def test_attention_part_prefill_then_decode(mode, window):
    hidden, heads, kv_heads, d = 72, 6, 2, 48
    rotary = RotarySpec(head_dim=d, rotary_dim=d, theta=777.0, max_positions=512)
    spec = AttentionSpec(hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=d, qkv_bias=True,
                         out_bias=False, scale=d ** -0.5, window=window, position=rotary)
    part = build_part(spec, "blk.attn.", mode)
    values = bind(part, mode, seed=3, scale=0.2)
    w = {k[len("blk.attn."):]: v for k, v in values.items()}
    cache = SequenceCache([part.cache_need()], 512, 512, part.act_dtype, DEV)
    assert part.cache_need() == KVNeed(kv_heads, d, window)
    part.prepare(DEV, cache.max_seq_len)
    stager = StepStager(DEV)
    rng = np.random.default_rng(4)
    lengths = [70, 5]
    xs = [torch.as_tensor(rng.standard_normal((n + 3, hidden))).to(part.act_dtype).to(DEV)
          for n in lengths]
    slots = cache.open(2)
    got = [[], []]
    # one prefill step for both, then three decode steps
    feeds = [[(0, lengths[0]), (0, lengths[1])]] + [[(lengths[0] + t, 1), (lengths[1] + t, 1)]
                                                    for t in range(3)]
    for feed in feeds:
        h = torch.cat([xs[i][a:a + n] for i, (a, n) in enumerate(feed)])
        ctx, ends = step_for(cache, stager, slots, [[0] * n for _, n in feed])
        residual = torch.zeros((h.shape[0], hidden), device=DEV)
        part.forward(h, ctx, cache.entry_view(0, ctx.tables), residual)
        cache.advance(slots, ends)
        at = 0
        for i, (_, n) in enumerate(feed):
            got[i].append(residual[at:at + n].double().cpu().numpy())
            at += n
    for i, n in enumerate(lengths):
        x = xs[i].double().cpu().numpy()
        want = plain.attention(x, w, heads, kv_heads, d, 777.0, np.arange(n + 3), window)
        close(np.concatenate(got[i]), want, mode, err_msg=f"sequence {i}")


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_mlp_part_adds_into_the_residual(mode):
    spec = GatedMLPSpec(hidden=88, intermediate=200, activation="silu")
    part = build_part(spec, "blk.mlp.", mode)
    values = bind(part, mode, seed=5, scale=0.2)
    w = {k[len("blk.mlp."):]: v for k, v in values.items()}
    h = (torch.randn(9, 88, device=DEV)).to(part.act_dtype)
    residual = torch.randn(9, 88, device=DEV)
    before = residual.double().cpu().numpy()
    part.forward(h, None, residual)
    want = before + plain.swiglu_mlp(h.double().cpu().numpy(), w)
    close(residual.double().cpu().numpy(), want, mode)


@pytest.mark.parametrize("n", [37, 150])
@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_block_part(mode, n):
    hidden, heads, kv_heads, d, inter = 64, 2, 1, 32, 144
    rotary = RotarySpec(head_dim=d, rotary_dim=d, theta=1e5, max_positions=256)
    norm = NormSpec(size=hidden, eps=1e-5)
    spec = BlockSpec(
        prefix="model.layers.0.",
        mixer=AttentionSpec(hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=d,
                            qkv_bias=True, out_bias=False, scale=d ** -0.5, window=None,
                            position=rotary),
        mixer_norm=norm, ffn=GatedMLPSpec(hidden=hidden, intermediate=inter, activation="silu"),
        ffn_norm=norm)
    part = build_part(spec, spec.prefix, mode)
    values = bind(part, mode, seed=6, scale=0.15)
    cache = SequenceCache([part.cache_need()], 256, 256, part.act_dtype, DEV)
    part.prepare(DEV, cache.max_seq_len)
    x = torch.randn(n, hidden, device=DEV)
    want = plain.decoder_layer(
        x.double().cpu().numpy(), values,
        {"hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
         "head_dim": d, "rms_norm_eps": 1e-5, "rope_theta": 1e5, "num_hidden_layers": 1}, 0,
        np.arange(n))
    (slot,) = cache.open(1)
    ctx, ends = step_for(cache, StepStager(DEV), [slot], [[0] * n])
    pending = part.forward(x, ctx, cache.entry_view(0, ctx.tables))
    # a block may hand back its last product for the next norm to add (a decode step's down
    # projection over a long K does); at these sizes every product is added where it is made:
    # by the own kernels' epilogue up to 64 tokens, by the library's (beta = 1) above
    assert pending is None
    close(x.double().cpu().numpy(), want, mode, factor=2.0)


def test_norm_part_adds_on_its_way():
    """`forward(x, add=delta)` leaves x + delta in x and returns the norm of the sum, bit for
    bit what the separate add and norm give; rows wider than the kernel keeps in registers
    too."""
    for size in (136, 1536, 4100, 4098):
        part = build_part(NormSpec(size=size, eps=1e-5), "some.norm", "bfloat16")
        bind(part, "bfloat16", scale=0.3)
        x = torch.randn(70, size, device=DEV) * 2
        delta = torch.randn(70, size, device=DEV)
        apart = x + delta
        want = part.forward(apart)
        got = part.forward(x, add=delta)
        assert torch.equal(x, apart) and torch.equal(got, want)
    fp32 = build_part(NormSpec(size=48, eps=1e-5), "some.norm", "float32")
    bind(fp32, "float32", scale=0.3)
    x = torch.randn(3, 48, device=DEV)
    delta = torch.randn(3, 48, device=DEV)
    apart = x + delta
    assert torch.equal(fp32.forward(x, add=delta), fp32.forward(apart)) and torch.equal(x, apart)


def test_unknown_kind_names_the_known_ones():
    class Spec:
        kind = "hyena"
    with pytest.raises(KeyError, match="gqa_attention"):
        build_part(Spec(), "x.", "float32")


def test_parts_refuse_sizes_the_kernels_do_not_take():
    rotary = RotarySpec(head_dim=24, rotary_dim=24, theta=1e4, max_positions=64)
    with pytest.raises(ValueError, match="multiples of 16"):
        build_part(AttentionSpec(hidden=48, heads=2, kv_heads=1, head_dim=24, qkv_bias=True,
                                 out_bias=False, scale=1.0, window=None, position=rotary),
                   "a.", "float32")
    with pytest.raises(ValueError, match="silu"):
        build_part(GatedMLPSpec(hidden=8, intermediate=8, activation="gelu"), "m.", "float32")

"""Safetensors files, the by-name check and the random-weights mode. No GPU."""

import json
import struct

import numpy as np
import pytest
import torch

import plain_model as plain
from semantic_aware_adaptive_kv_cache_precision_b200.engine.model import DecoderModel
from semantic_aware_adaptive_kv_cache_precision_b200.config import Qwen2Config
from semantic_aware_adaptive_kv_cache_precision_b200.weights import (
    Checkpoint, SafetensorsFile, TensorDecl, WeightArena, WeightError, check_tensors,
    device_dtype, load_checkpoint, write_random_model, write_safetensors)
from conftest import TINY_A, TINY_B


def test_round_trip_all_stored_types(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(4).to(torch.bfloat16),
               "c": torch.randn(2, 2).to(torch.float16), "d": torch.arange(6, dtype=torch.int32),
               "e": torch.empty(0, 3)}
    write_safetensors(tmp_path / "m.safetensors", tensors, {"note": 1})
    f = SafetensorsFile(tmp_path / "m.safetensors")
    assert set(f.infos) == set(tensors)
    for name, t in tensors.items():
        got = f.tensor(name)
        assert got.dtype == t.dtype and tuple(got.shape) == tuple(t.shape)
        assert torch.equal(got, t)
    # the independent reader of the plain implementation agrees
    other = plain.read_safetensors(tmp_path / "m.safetensors")
    np.testing.assert_array_equal(other["b"], tensors["b"].double().numpy())


def test_broken_files_are_named(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 10 ** 12) + b"{}")
    with pytest.raises(WeightError, match="announce a header"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(WeightError, match="not JSON"):
        SafetensorsFile(p)
    write_safetensors(p, {"w": torch.randn(8, 8)})
    data = p.read_bytes()
    p.write_bytes(data[:-40])
    with pytest.raises(WeightError, match="cut short"):
        SafetensorsFile(p)
    header = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0\0")
    with pytest.raises(WeightError, match="F8_E4M3 is not supported"):
        SafetensorsFile(p)


def _decls(raw):
    return DecoderModel.tensor_decls_of(Qwen2Config.from_dict(raw).model_spec())


def test_expected_tensors_follow_the_config():
    names = {d.name: tuple(d.shape) for d in _decls(TINY_A)}
    assert names["model.embed_tokens.weight"] == (512, 64)
    assert names["model.layers.1.self_attn.k_proj.weight"] == (32, 64)
    assert names["model.layers.0.self_attn.q_proj.bias"] == (64,)
    assert names["model.layers.0.mlp.down_proj.weight"] == (64, 176)
    assert "model.layers.0.self_attn.o_proj.bias" not in names
    assert "lm_head.weight" not in names and len(names) == 1 + 2 * 12 + 1
    assert _decls(TINY_B)[-1].name == "lm_head.weight"


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    folder = write_random_model(tmp_path / "m", dict(TINY_A), 0)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.infos}
    del tensors["model.norm.weight"]
    del tensors["model.layers.1.mlp.up_proj.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(64, 176)
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightError) as err:
        load_checkpoint(folder, _decls(TINY_A), "float32", "cpu")
    text = str(err.value)
    assert "2 missing, 1 unexpected, 1 wrong" in text and "nothing was allocated" in text
    for piece in ("model.norm.weight: missing", "up_proj.weight: missing",
                  "rotary_emb.inv_freq: unexpected", "gate_proj.weight: shape (64, 176)"):
        assert piece in text


def test_nan_is_refused_by_name(tmp_path):
    folder = write_random_model(tmp_path / "m", dict(TINY_A), 0)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.infos}
    tensors["model.layers.0.self_attn.v_proj.bias"][3] = float("nan")
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightError, match="v_proj.bias: holds NaN"):
        load_checkpoint(folder, _decls(TINY_A), "float32", "cpu")


def test_types_on_the_device():
    assert device_dtype("BF16", "bfloat16") == torch.bfloat16
    assert device_dtype("F16", "bfloat16") == torch.bfloat16
    assert device_dtype("F32", "bfloat16") == torch.float32      # stored in 32 bits: stays so
    assert device_dtype("I64", "bfloat16") == torch.int32
    for stored in ("BF16", "F16", "F32"):
        assert device_dtype(stored, "float32") == torch.float32
    with pytest.raises(ValueError):
        device_dtype("F32", "float16")


def test_arena_lays_groups_back_to_back(tmp_path):
    folder = write_random_model(tmp_path / "m", dict(TINY_B), 1, dtype="bfloat16")
    decls = _decls(TINY_B)
    arena = load_checkpoint(folder, decls, "bfloat16", "cpu")
    f = SafetensorsFile(folder / "model.safetensors")
    p = "model.layers.2.self_attn."
    qkv = arena.group_view(p + "qkv.weight")
    assert qkv.shape == (192 + 2 * 32, 192) and qkv.dtype == torch.bfloat16
    assert torch.equal(qkv[:192], f.tensor(p + "q_proj.weight"))
    assert torch.equal(qkv[192:224], f.tensor(p + "k_proj.weight"))
    assert torch.equal(qkv[224:], f.tensor(p + "v_proj.weight"))
    assert torch.equal(arena.group_view(p + "qkv.bias")[192:224], f.tensor(p + "k_proj.bias"))
    for name, offset in arena.offsets.items():
        d = arena.decls[name]
        if d.group is None or name.endswith("q_proj.weight") or name.endswith("q_proj.bias") \
                or name.endswith("gate_proj.weight"):
            assert offset % 256 == 0
    # mixed stored types cannot be joined: the group view says so
    mixed = [TensorDecl("a", (2, 4), group="g"), TensorDecl("b", (2, 4), group="g")]
    arena2 = WeightArena(mixed, {"a": torch.float32, "b": torch.bfloat16}, "cpu")
    assert arena2.group_view("g") is None or arena2.group_view("g").shape[0] == 2


def test_random_model_is_a_function_of_seed_and_name(tmp_path):
    a = write_random_model(tmp_path / "a", dict(TINY_A), 0)
    b = write_random_model(tmp_path / "b", dict(TINY_A), 0)
    c = write_random_model(tmp_path / "c", dict(TINY_A), 1)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    config, tensors = plain.read_model_folder(a)
    assert config["architectures"] == ["Qwen2ForCausalLM"] and config["hidden_size"] == 64
    norm = tensors["model.layers.0.input_layernorm.weight"]
    assert abs(norm.mean() - 1.0) < 0.02 and 0.005 < norm.std() < 0.04
    w = tensors["model.layers.1.mlp.down_proj.weight"]
    assert abs(w.mean()) < 0.002 and abs(w.std() - 0.02) < 0.002
    assert abs(tensors["model.layers.0.self_attn.k_proj.bias"].std() - 0.02) < 0.01
    check_tensors(Checkpoint(a), _decls(TINY_A), "config.json")


def test_a_checkpoint_in_two_shards_loads_like_one_file(tmp_path):
    """`model.safetensors.index.json` names the shard of every tensor; the loader finds
    each tensor in its shard and the arena is the one a single file gives."""
    whole = write_random_model(tmp_path / "whole", dict(TINY_B), 1, dtype="bfloat16")
    f = SafetensorsFile(whole / "model.safetensors")
    names = list(f.infos)
    halves = {"model-00001-of-00002.safetensors": names[:len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    (sharded / "config.json").write_text((whole / "config.json").read_text())
    weight_map = {}
    for shard, members in halves.items():
        write_safetensors(sharded / shard, {n: f.tensor(n) for n in members})
        weight_map.update({n: shard for n in members})
    (sharded / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {}, "weight_map": weight_map}))
    decls = _decls(TINY_B)
    one = load_checkpoint(whole, decls, "bfloat16", "cpu")
    two = load_checkpoint(sharded, decls, "bfloat16", "cpu")
    assert one.offsets == two.offsets
    assert all(torch.equal(one.view(d.name), two.view(d.name)) for d in decls)
    # a tensor missing from its shard is named like any other missing tensor
    del two
    (sharded / "model-00002-of-00002.safetensors").unlink()
    write_safetensors(sharded / "model-00002-of-00002.safetensors",
                      {n: f.tensor(n) for n in halves["model-00002-of-00002.safetensors"][1:]})
    with pytest.raises(WeightError, match="1 missing"):
        load_checkpoint(sharded, decls, "bfloat16", "cpu")
    # a folder with neither a file nor an index says so
    (tmp_path / "empty").mkdir()
    with pytest.raises(WeightError, match="neither"):
        Checkpoint(tmp_path / "empty")


def test_names_an_architecture_lets_pass_are_not_unexpected(tmp_path):
    folder = write_random_model(tmp_path / "m", dict(TINY_A), 0)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.infos}     # the file is rewritten below
    del f
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    tensors["model.layers.0.self_attn.stray"] = torch.ones(2)
    write_safetensors(folder / "model.safetensors", tensors)
    spec = Qwen2Config.from_dict(TINY_A).model_spec()
    assert spec.ignore_tensors == ("*.rotary_emb.inv_freq",)
    with pytest.raises(WeightError) as err:
        load_checkpoint(folder, _decls(TINY_A), "float32", "cpu", ignore=spec.ignore_tensors)
    assert "1 unexpected" in str(err.value) and "stray" in str(err.value)
    assert "inv_freq" not in str(err.value)
    with pytest.raises(WeightError, match="2 unexpected"):
        load_checkpoint(folder, _decls(TINY_A), "float32", "cpu")


def test_an_arena_the_device_cannot_hold_is_a_typed_error(tmp_path, monkeypatch):
    """The allocator's failure comes back as `OutOfDeviceMemory` that says what was asked
    for (`tests/test_emergency_downgrade.py:40-54` of the reference injects the same way)."""
    from semantic_aware_adaptive_kv_cache_precision_b200 import OutOfDeviceMemory
    folder = write_random_model(tmp_path / "m", dict(TINY_A), 0)
    real = torch.empty

    def no_room(*args, **kwargs):
        if kwargs.get("dtype") == torch.uint8:
            raise torch.OutOfMemoryError("injected")
        return real(*args, **kwargs)

    monkeypatch.setattr(torch, "empty", no_room)
    with pytest.raises(OutOfDeviceMemory, match="the model's weights"):
        load_checkpoint(folder, _decls(TINY_A), "float32", "cpu")

"""Model folders: safetensors round trip, the one error that lists everything wrong, the dtype
rule, the random-weights mode."""

import json
import struct

import pytest
import torch

from gtar_kimik3_public_b200.models import Model
from gtar_kimik3_public_b200.registry import architecture, config_from_dict
from gtar_kimik3_public_b200.weights import (ModelFolderTensors, SafetensorsError, WeightsError, load_weights,
                                             write_random_model, write_safetensors)
from tests.plain.weights import read_safetensors, tensor_names
from tests.tiny_configs import TINY_A, TINY_B


def _model(cfg_dict, dtype=torch.bfloat16):
    config = config_from_dict(cfg_dict)
    return Model(architecture(config.ARCH_NAMES[0]).build_plan(config), config, dtype, "cpu")


def test_round_trip_keeps_bits_and_alignment(tmp_path):
    tensors = {
        "a": torch.randn(3, 5).to(torch.bfloat16),  # odd element count before a float32 tensor
        "b": torch.randn(7),
        "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
        "d": torch.randn(2, 2, dtype=torch.float64),
    }
    write_safetensors(tmp_path / "model.safetensors", tensors, {"note": "x"})
    folder = ModelFolderTensors(tmp_path)
    assert set(folder.names()) == set(tensors)
    for name, want in tensors.items():
        got = folder.tensor(name)
        assert got.dtype == want.dtype and torch.equal(got, want)
    mine = read_safetensors(tmp_path / "model.safetensors")  # the tests' own reader agrees
    assert torch.equal(mine["a"], tensors["a"].float())


def test_random_model_names_match_the_reference_state_dict(tmp_path):
    for cfg in (TINY_A, TINY_B):
        folder = write_random_model(tmp_path / cfg["head_dim"].__str__(), config_from_dict(cfg), seed=0)
        have = ModelFolderTensors(folder)
        want = {name: shape for name, shape, _ in tensor_names(cfg)}
        assert {n: have.shape(n) for n in have.names()} == want
        assert json.loads((folder / "config.json").read_text())["head_dim"] == cfg["head_dim"]
        assert have.dtype("model.embed_tokens.weight") == torch.bfloat16
        assert have.dtype("model.norm.weight") == torch.float32


def test_random_weights_are_a_function_of_the_seed(tmp_path):
    config = config_from_dict(TINY_B)
    a = read_safetensors(write_random_model(tmp_path / "a", config, 5) / "model.safetensors")
    b = read_safetensors(write_random_model(tmp_path / "b", config, 5) / "model.safetensors")
    c = read_safetensors(write_random_model(tmp_path / "c", config, 6) / "model.safetensors")
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    norm = a["model.layers.0.self_attn.q_norm.weight"]
    assert 0.5 < norm.mean() < 1.5 and norm.std() > 0.01  # not all ones: a dropped norm weight would show


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(tmp_path, config_from_dict(TINY_B), 0)
    tensors = {n: ModelFolderTensors(folder).tensor(n).clone() for n in ModelFolderTensors(folder).names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(4)
    tensors["model.layers.2.self_attn.k_norm.weight"] = torch.zeros(31)
    tensors["lm_head.weight"] = tensors["lm_head.weight"].T.contiguous()
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as err:
        load_weights(_model(TINY_B), folder)
    e = err.value
    assert sorted(e.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert sorted(n for n, _, _ in e.wrong_shape) == ["lm_head.weight", "model.layers.2.self_attn.k_norm.weight"]
    text = str(e)
    for name in e.missing + e.unexpected:
        assert name in text
    assert "[31]" in text and "expected [32]" in text


def test_dtype_rule(tmp_path):
    config = config_from_dict(TINY_A)
    folder = write_random_model(tmp_path, config, 0)
    tensors = {n: ModelFolderTensors(folder).tensor(n).clone() for n in ModelFolderTensors(folder).names()}
    # one projection stored in 32-bit: it stays so in a bfloat16 run
    tensors["model.layers.0.self_attn.o_proj.weight"] = tensors["model.layers.0.self_attn.o_proj.weight"].float()
    tensors["model.layers.1.input_layernorm.weight"] = tensors["model.layers.1.input_layernorm.weight"].to(torch.bfloat16)
    write_safetensors(folder / "model.safetensors", tensors)
    bf16 = _model(TINY_A, torch.bfloat16)
    load_weights(bf16, folder)
    layers = bf16.plan.layers
    assert layers[0].mixer.w_o.dtype == torch.float32
    assert layers[1].mixer.w_o.dtype == torch.bfloat16
    assert layers[0].mixer.w_qkv.dtype == torch.bfloat16 and layers[0].mixer.w_qkv.shape == (4 * 16 + 2 * 2 * 16, 64)
    assert layers[0].input_norm.weight.dtype == torch.float32
    assert layers[1].input_norm.weight.dtype == torch.bfloat16
    assert bf16.plan.head.weight is bf16.plan.embedding.weight  # tied
    f32 = _model(TINY_A, torch.float32)
    load_weights(f32, folder)
    assert all(t.dtype == torch.float32 for t in (f32.plan.layers[1].mixer.w_qkv, f32.plan.layers[1].input_norm.weight,
                                                   f32.plan.embedding.weight))
    # packing: q | k | v one after another; gate and up rows alternate
    packed = f32.plan.layers[1].feed_forward.w_gate_up
    assert torch.equal(packed[0::2], tensors["model.layers.1.mlp.gate_proj.weight"].float())
    assert torch.equal(packed[1::2], tensors["model.layers.1.mlp.up_proj.weight"].float())
    qkv = f32.plan.layers[1].mixer.w_qkv
    assert torch.equal(qkv[:64], tensors["model.layers.1.self_attn.q_proj.weight"].float())
    assert torch.equal(qkv[64:96], tensors["model.layers.1.self_attn.k_proj.weight"].float())
    assert torch.equal(qkv[96:], tensors["model.layers.1.self_attn.v_proj.weight"].float())


def test_tied_model_accepts_a_stored_head(tmp_path):
    folder = write_random_model(tmp_path, config_from_dict(TINY_A), 0)
    tensors = {n: ModelFolderTensors(folder).tensor(n).clone() for n in ModelFolderTensors(folder).names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()  # the reference's state dict has it
    write_safetensors(folder / "model.safetensors", tensors)
    load_weights(_model(TINY_A), folder)


def test_truncated_and_malformed_files(tmp_path):
    folder = write_random_model(tmp_path, config_from_dict(TINY_A), 0)
    path = folder / "model.safetensors"
    data = path.read_bytes()
    path.write_bytes(data[: len(data) // 2])
    with pytest.raises(SafetensorsError, match="truncated"):
        ModelFolderTensors(folder)
    path.write_bytes(struct.pack("<Q", 10**9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        ModelFolderTensors(folder)
    path.unlink()
    with pytest.raises(FileNotFoundError):
        ModelFolderTensors(folder)

"""The converter from the reference's checkpoint files (src/common.py:85-93) to model folders: a tiny checkpoint,
written by the reference's own ``save_checkpoint`` where a copy of the reference is at hand (else by ``torch.save``
of the same dictionary), becomes a folder whose tensors are the checkpoint's and from which the plain
implementation, and on a GPU the engine, generates the greedy tokens stored under tests/golden/."""

import dataclasses
import json
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.plain import model as plain
from tests.plain.weights import make_weights, read_safetensors
from tests.tiny_configs import TINY_A, TINY_B

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = Path(__file__).parent / "golden"
REFERENCE_FIELDS = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings", "initializer_range")


def reference_folder():
    for folder in (os.environ.get("GTAR_REFERENCE_DIR"), ROOT / "baseline" / "_ref"):
        if folder and (Path(folder) / "src" / "common.py").exists():
            return Path(folder)
    return None


def write_checkpoint(path: Path, cfg: dict, seed: int) -> dict:
    """A checkpoint in the reference's format holding the golden files' weights; returns those weights."""
    weights = make_weights(cfg, seed, std=0.08)
    state = dict(weights)
    if cfg["tie_word_embeddings"]:
        state["lm_head.weight"] = state["model.embed_tokens.weight"]  # the reference's state dict lists the tied head too
    fields = {k: cfg[k] for k in REFERENCE_FIELDS}
    folder = reference_folder()
    if folder is not None:
        sys.dont_write_bytecode = True
        sys.path.insert(0, str(folder))
        try:
            from src.common import save_checkpoint
            from src.models import ARCHITECTURES
        finally:
            sys.path.remove(str(folder))
        config_class, model_class = ARCHITECTURES["transformer"]
        model = model_class(config_class(**fields))
        model.load_state_dict(state, strict=True)

        class Loader:
            def state_dict(self):
                return {"position": 0}

        save_checkpoint(path, model, torch.optim.SGD(model.parameters(), lr=0.1), Loader(), 7, config_class(**fields))
    else:
        torch.save({"model": state, "optimizer": {}, "loader": {"position": 0}, "step": 7, "config": fields}, path)
    return weights


@pytest.mark.parametrize("tag,cfg,seed", [("tiny_a", TINY_A, 0), ("tiny_b", TINY_B, 1)])
def test_converted_folder_holds_the_checkpoint_and_generates_the_golden_tokens(tmp_path, tag, cfg, seed):
    from gtar_kimik3_public_b200.registry import config_from_file
    from gtar_kimik3_public_b200.weights.convert import convert_checkpoint

    weights = write_checkpoint(tmp_path / "ckpt.pt", cfg, seed)
    folder = convert_checkpoint(tmp_path / "ckpt.pt", tmp_path / "model", extra_config={"max_position_embeddings": cfg["max_position_embeddings"]})
    config = config_from_file(folder)
    assert dataclasses.asdict(config)["hidden_size"] == cfg["hidden_size"] and config.max_position_embeddings == cfg["max_position_embeddings"]
    stored = read_safetensors(folder / "model.safetensors")
    for name, tensor in weights.items():
        assert stored[name].dtype == torch.float32 and torch.equal(stored[name], tensor), name
    data = np.load(GOLDEN / f"{tag}.npz")
    for r in range(3):
        want = data[f"greedy_{r}"].tolist()
        assert plain.greedy_generate(data[f"ids_{r}"].tolist(), stored, cfg, len(want)) == want


def test_converter_reports_what_does_not_fit(tmp_path):
    from gtar_kimik3_public_b200.weights import WeightsError
    from gtar_kimik3_public_b200.weights.convert import convert_checkpoint

    weights = make_weights(TINY_A, 0, std=0.08)
    state = {k: v for k, v in weights.items() if "k_norm" not in k}
    state["model.layers.0.extra.weight"] = torch.zeros(3)
    torch.save({"model": state, "config": {k: TINY_A[k] for k in REFERENCE_FIELDS}}, tmp_path / "bad.pt")
    with pytest.raises(WeightsError) as error:
        convert_checkpoint(tmp_path / "bad.pt", tmp_path / "model")
    assert "k_norm" in str(error.value) and "extra" in str(error.value)
    torch.save({"weights": {}}, tmp_path / "other.pt")
    with pytest.raises(ValueError):
        convert_checkpoint(tmp_path / "other.pt", tmp_path / "model")


@pytest.mark.gpu
@pytest.mark.parametrize("tag,cfg,seed", [("tiny_a", TINY_A, 0), ("tiny_b", TINY_B, 1)])
def test_engine_generates_the_golden_tokens_from_a_converted_checkpoint(tmp_path, tag, cfg, seed):
    from gtar_kimik3_public_b200 import generate as api
    from gtar_kimik3_public_b200.weights.convert import convert_checkpoint

    write_checkpoint(tmp_path / "ckpt.pt", cfg, seed)
    folder = convert_checkpoint(tmp_path / "ckpt.pt", tmp_path / "model", extra_config={"max_position_embeddings": cfg["max_position_embeddings"]})
    model = api.load(folder, "float32", "cuda:0")
    data = np.load(GOLDEN / f"{tag}.npz")
    prompts = [data[f"ids_{r}"].tolist() for r in range(3)]
    want = [data[f"greedy_{r}"].tolist() for r in range(3)]
    got = api.generate(model, prompts, max_new_tokens=len(want[0]), temperature=0.0)
    assert got == want


def test_converter_command_line(tmp_path, capsys):
    from gtar_kimik3_public_b200.registry import config_from_file
    from gtar_kimik3_public_b200.weights import convert

    write_checkpoint(tmp_path / "ckpt.pt", TINY_B, 1)
    assert convert.main([str(tmp_path / "ckpt.pt"), str(tmp_path / "model"), "--dtype", "bfloat16", "--max-position-embeddings", "256",
                         "--eos-token-id", "7"]) == 0
    assert "model.safetensors" in capsys.readouterr().out
    config = config_from_file(tmp_path / "model")
    assert config.max_position_embeddings == 256 and config.eos_token_id == 7
    stored = read_safetensors(tmp_path / "model" / "model.safetensors")
    assert stored["lm_head.weight"].shape == (TINY_B["vocab_size"], TINY_B["hidden_size"])
    weights = make_weights(TINY_B, 1, std=0.08)  # values bfloat16 holds exactly, so rounding the matrices changed nothing
    assert torch.equal(stored["model.layers.1.mlp.up_proj.weight"], weights["model.layers.1.mlp.up_proj.weight"])

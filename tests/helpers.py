"""Shared pieces of the tests: tiny model folders in temporary places, the plain logits of a
request, and the bfloat16 error yardstick."""

from __future__ import annotations

import functools
import tempfile
from pathlib import Path

import torch

from tests.plain import model as plain
from tests.plain.weights import read_safetensors
from tests.tiny_configs import REAL_06B, REAL_4B, REAL_8B, TINY_A, TINY_B, TINY_C, TINY_LONG

CONFIGS = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_long": TINY_LONG,
           "real_06b": REAL_06B, "real_4b": REAL_4B, "real_8b": REAL_8B}
WEIGHT_STD = 0.08  # wide enough that logits are O(1) and an error of 1e-3 is an error
# at real widths the reference's own 0.02 gives logits of size O(1) (sqrt(1024) * 0.02 = 0.64)
STD_OF = {"real_06b": 0.03, "real_4b": 0.02, "real_8b": 0.016}
# where the plain implementation runs: the real sizes and the long sequences would take minutes on the CPU
PLAIN_DEVICE = {"real_06b": "cuda", "real_4b": "cuda", "real_8b": "cuda", "tiny_long": "cuda"}

_folders: dict[tuple, tempfile.TemporaryDirectory] = {}


def model_folder(tag: str, seed: int = 0, std: float | None = None) -> Path:
    """A folder with config.json and model.safetensors for one of the tiny configurations, written
    by the library's random-weights mode into a temporary directory (kept for the session)."""
    std = STD_OF.get(tag, WEIGHT_STD) if std is None else std
    key = (tag, seed, std)
    if key not in _folders:
        from gtar_kimik3_public_b200.registry import config_from_dict
        from gtar_kimik3_public_b200.weights import write_random_model

        holder = tempfile.TemporaryDirectory(prefix=f"gtar_test_{tag}_")
        write_random_model(holder.name, config_from_dict(CONFIGS[tag]), seed, std=std)
        _folders[key] = holder
    return Path(_folders[key].name)


@functools.lru_cache(maxsize=None)
def plain_weights(tag: str, seed: int = 0, std: float | None = None):
    weights = read_safetensors(model_folder(tag, seed, std) / "model.safetensors")
    device = PLAIN_DEVICE.get(tag, "cpu")
    return weights if device == "cpu" else {name: tensor.to(device) for name, tensor in weights.items()}


def requests_for(tag: str, lengths, seed: int = 7) -> list[list[int]]:
    gen = torch.Generator().manual_seed(seed)
    vocab = CONFIGS[tag]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lengths]


_plain_cache: dict = {}


def plain_logits(tag: str, tokens: list[int], mode: str = "f64", seed: int = 0) -> torch.Tensor:
    """Logits [T, V] of the plain implementation: ``f64`` (the oracle), ``f32``, or ``lowp`` (float32
    with every matrix product rounded to bfloat16, as the reference computes under autocast)."""
    key = (tag, tuple(tokens), mode, seed)
    if key not in _plain_cache:
        weights = plain_weights(tag, seed)
        ids = torch.tensor(tokens)
        if mode == "f64":
            out = plain.forward(ids, weights, CONFIGS[tag], torch.float64)
        elif mode == "f32":
            out = plain.forward(ids, weights, CONFIGS[tag], torch.float32)
        else:
            plain.LOWP = torch.bfloat16
            try:
                out = plain.forward(ids, weights, CONFIGS[tag], torch.float32)
            finally:
                plain.LOWP = None
        _plain_cache[key] = out.cpu()
    return _plain_cache[key]


def load_engine(tag: str, dtype: str, max_tokens: int, seed: int = 0, max_seqs: int | None = None, **options):
    from gtar_kimik3_public_b200.engine import Engine
    from gtar_kimik3_public_b200.generate import load

    model = load(model_folder(tag, seed), dtype, "cuda:0")
    return Engine(model, max_tokens, max_seqs=max_seqs, **options)


def poison(engine) -> None:
    """Fills every page with NaN so that a read of a place no step has written shows in the logits."""
    for group in engine.cache.kv_groups:
        group.k.fill_(float("nan"))
        group.v.fill_(float("nan"))


def check_against_plain(tag: str, dtype: str, tokens: list[int], places: list[int], got: torch.Tensor, what: str) -> None:
    """``got[i]`` are the engine's logits at ``places[i]`` of the request ``tokens``.

    float32: within 1e-4 of the float64 oracle on logits of size O(1) (the reference's own
    float32 test allows 1e-3, tests/test_inference.py:34).  bfloat16: the reference's rule for a
    low-precision kernel, tests/test_flash_attention_2.py:54-58: our error against the oracle may be
    at most twice the error of a standard low-precision implementation plus 1e-4 — the
    standard here being the plain implementation with bfloat16 matrix products.
    """
    got = got.detach().double().cpu()
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    oracle = plain_logits(tag, tokens, "f64")[places]
    err = (got - oracle).abs().max().item()
    if dtype == "float32":
        assert err < 1e-4, f"{what}: float32 logits differ from the oracle by {err:.3e}"
    else:
        lowp = plain_logits(tag, tokens, "lowp")[places].double()
        yard = (lowp - oracle).abs().max().item()
        assert err <= 2 * yard + 1e-4, f"{what}: bfloat16 error {err:.3e} exceeds twice the yardstick {yard:.3e}"

"""The plain implementation against the reference's own model code (outputs stored once under
tests/golden/, made by tests/golden/make_golden.py from qtris123/gtar-kimik3-public's
src/models/transformer.py and src/engine.py on the CPU in float32)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from tests.plain import model as plain
from tests.plain.weights import make_weights
from tests.tiny_configs import TINY_A, TINY_B

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("tag,cfg,seed", [("tiny_a", TINY_A, 0), ("tiny_b", TINY_B, 1)])
def test_plain_matches_reference_logits(tag, cfg, seed):
    data = np.load(GOLDEN / f"{tag}.npz")
    weights = make_weights(cfg, seed, std=0.08)
    for r in range(3):
        ids = torch.from_numpy(data[f"ids_{r}"])
        want = torch.from_numpy(data[f"logits_{r}"])
        got = plain.forward(ids, weights, cfg)
        assert got.shape == want.shape
        # the reference's own cut-to-cut wobble in float32 is 4.8e-7 on logits of this size
        assert (got - want).abs().max().item() < 2e-5, (tag, r)
        assert want.abs().max().item() > 0.5  # the comparison is not between near-zero numbers


@pytest.mark.parametrize("tag,cfg,seed", [("tiny_a", TINY_A, 0), ("tiny_b", TINY_B, 1)])
def test_plain_matches_reference_greedy(tag, cfg, seed):
    data = np.load(GOLDEN / f"{tag}.npz")
    weights = make_weights(cfg, seed, std=0.08)
    for r in range(3):
        want = data[f"greedy_{r}"].tolist()
        got = plain.greedy_generate(data[f"ids_{r}"].tolist(), weights, cfg, len(want))
        assert got == want, (tag, r)


def test_plain_float64_agrees_with_float32():
    weights = make_weights(TINY_B, 3, std=0.08)
    ids = torch.randint(0, TINY_B["vocab_size"], (23,), generator=torch.Generator().manual_seed(5))
    a = plain.forward(ids, weights, TINY_B, torch.float32)
    b = plain.forward(ids, weights, TINY_B, torch.float64)
    assert (a.double() - b).abs().max().item() < 1e-4

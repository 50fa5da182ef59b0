"""Token choice on the device, with the reference's options (src/engine.py:5-12):
``temperature == 0`` is greedy; otherwise logits are divided by the temperature, optionally cut to
the ``top_k`` largest (ties at the threshold survive), and one token is drawn from the softmax.
The draw is keyed by (seed, request, step) instead of a global generator, so a request's tokens do
not depend on what else is in the batch; see the kernel file for the rule.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import functional as F


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0  # the reference's API default (src/engine.py:26)
    top_k: int | None = None  # None or 0: off (src/engine.py:27)
    seed: int = 42  # the reference's command-line default (scripts/generate.py:28)

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0 (0 = greedy)")
        if self.top_k is not None and self.top_k < 0:
            raise ValueError("top_k must be >= 0")


def choose(logits: torch.Tensor, params: SamplingParams, request_ids: torch.Tensor | None, steps: torch.Tensor | None,
           advance_steps: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of ``logits`` (float32 ``[n, vocab]``) as int32 on the device.  Greedy choice
    (temperature 0) reads neither ``request_ids`` nor ``steps``."""
    if params.temperature == 0:
        return F.argmax(logits, out)
    return F.sample(logits, params.temperature, params.top_k or 0, params.seed, request_ids, steps, advance_steps, out)

"""Token embedding (``h0 = E[ids]``, src/models/transformer.py:55,61) and the output head
(``logits = z @ W.T``, tied to the embedding table or its own; transformer.py:75-77,101)."""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.linear import linear
from .base import Part, TensorSpec


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return F.embed_rows(self.weight, ids)


class OutputHead(Part):
    graph_safe = True

    """Logits in float32.  ``tied_to`` names an embedding whose table is used instead of an own matrix."""

    def __init__(self, hidden_size: int, vocab_size: int, tied_to: TokenEmbedding | None = None):
        self.hidden_size, self.vocab_size, self.tied_to = int(hidden_size), int(vocab_size), tied_to
        self._weight: torch.Tensor | None = None

    def tensor_specs(self):
        # A tied model's file may still carry the head (the reference's state dict does): it is
        # accepted and not read.
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied_to is not None)}

    def load(self, tensors):
        if self.tied_to is None:
            self._weight = tensors["weight"].contiguous()

    @property
    def weight(self) -> torch.Tensor:
        return self.tied_to.weight if self.tied_to is not None else self._weight

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        return linear(z, self.weight, torch.float32)

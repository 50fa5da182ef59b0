"""RMSNorm: ``weight * (x * rsqrt(mean(x^2) + eps))`` in 32-bit (src/layers/rmsnorm.py:11-16),
fused with the add of a pending branch output into the residual stream."""

from __future__ import annotations

import torch

from ..ops import functional as F
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), "vector")}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def decode_record(self):
        return {"kind": "rmsnorm", "size": self.size, "eps": self.eps, "weight": self.weight}

    def forward(self, h, delta, out_dtype, rows=None):
        return F.add_rmsnorm(h, delta, self.weight, self.eps, out_dtype, rows)


register_part("norm", "rmsnorm", RMSNorm)

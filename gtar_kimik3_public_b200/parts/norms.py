"""RMSNorm: ``weight * (x * rsqrt(mean(x^2) + eps))`` in 32-bit (src/layers/rmsnorm.py:11-16),
fused with the add of a pending branch output into the residual stream."""

from __future__ import annotations

import torch

from ..ops import functional as F
from .base import DeferredProjection, Norm, TensorSpec, register_part


class RMSNorm(Norm):
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

    takes_deferred = True

    def forward(self, h, delta, out_dtype, rows=None, prescaled_ok=False):
        if isinstance(delta, DeferredProjection):
            x, w = delta.x, delta.weight
            if (prescaled_ok and rows is None and out_dtype == torch.bfloat16 and h.dtype == torch.float32
                    and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= F.SKINNY_M
                    and x.shape[1] % 8 == 0 and h.shape[1] % 8 == 0):
                # few tokens: the projection adds into the stream and leaves the rows times this norm's weight;
                # the division by the root mean square happens where the next product is written
                return F.gemm_tc_residual(x, w, h, self.weight, self.eps)
            delta = delta.materialize()
        return F.add_rmsnorm(h, delta, self.weight, self.eps, out_dtype, rows)


register_part("norm", "rmsnorm", RMSNorm)

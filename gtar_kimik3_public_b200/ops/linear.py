"""The matrix product of a projection, ``y = x @ W.T`` (no bias; src/layers/attention.py:62-65).

The kernel is chosen by the weight's dtype: a float32 weight always goes through the FP32-pipe
kernel (true 32-bit: no tensor cores, no TF32), whatever the activations are; a bfloat16 weight
goes through the tensor-core product with 32-bit accumulation.
"""

from __future__ import annotations

import torch

from . import functional as F
from .library import KernelError, require_device


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x [M, K] @ weight[N, K].T -> [M, N]`` in ``out_dtype`` (default: ``x.dtype``)."""
    require_device(x.device)
    out_dtype = out_dtype or x.dtype
    if weight.dtype == torch.float32:
        return F.linear_f32(x, weight, out_dtype)
    if weight.dtype != torch.bfloat16:
        raise KernelError(f"projection weights are float32 or bfloat16, not {weight.dtype}")
    if x.dtype != torch.bfloat16:
        raise KernelError("a bfloat16 weight needs bfloat16 activations")
    return F.linear_bf16(x, weight, out_dtype)

"""The matrix product of a projection, ``y = x @ W.T`` (no bias; src/layers/attention.py:62-65).

The kernel is chosen by the weight's dtype: a float32 weight always goes through the FP32-pipe
kernel (true 32-bit: no tensor cores, no TF32), whatever the activations are; a bfloat16 weight
goes through the tcgen05 tensor-core kernel with 32-bit accumulation (or, for shapes it does not
take, the library product the reference itself uses).
"""

from __future__ import annotations

import torch

from . import functional as F
from .library import KernelError, require_device


def _tc_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned rows: k a multiple of 8 elements."""
    return x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None,
           swiglu: bool = False) -> torch.Tensor:
    """``x [M, K] @ weight[N, K].T -> [M, N]`` in ``out_dtype`` (default: ``x.dtype``).

    ``swiglu``: ``weight`` holds gate and up rows alternately and the result is ``silu(gate) * up``
    of width ``N / 2``.
    """
    require_device(x.device)
    out_dtype = out_dtype or x.dtype
    if weight.dtype == torch.float32:
        y = F.linear_f32(x, weight, torch.float32 if swiglu else out_dtype)
        return F.swiglu(y, interleaved=True).to(out_dtype) if swiglu else y
    if weight.dtype != torch.bfloat16:
        raise KernelError(f"projection weights are float32 or bfloat16, not {weight.dtype}")
    if x.dtype != torch.bfloat16:
        raise KernelError("a bfloat16 weight needs bfloat16 activations")
    if not _tc_ok(x, weight):
        y = F.linear_bf16(x, weight, torch.bfloat16 if swiglu else out_dtype)
        return F.swiglu(y, interleaved=True) if swiglu else y
    if F.gemv_suits(x.shape[0], weight.shape[0], x.shape[1], x.device):
        return F.gemv(x, weight, torch.bfloat16 if swiglu else out_dtype, swiglu=swiglu)
    splits = F.split_k_for(x.shape[0], weight.shape[0], x.shape[1])
    return F.gemm_tc(x, weight, torch.bfloat16 if swiglu else out_dtype, swiglu=swiglu, splits=splits)

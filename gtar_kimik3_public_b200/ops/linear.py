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


# Most tokens for which ``linear_after_norm`` uses the product that normalises its own input.  Measured inside a
# decode step (28 layers of width 1024, batch 8) the folded kernel took 20 to 25 us against 3.5 us for the norm
# kernel plus 11 us for the plain product, because each of its ~128 blocks reads the tokens' whole rows before
# its first MMA; so it is off (0) and the norm runs as a kernel of its own.  ``F.NORMED_MAX_TOKENS`` turns it on.
FOLD_NORM_MAX_TOKENS = 0


def linear_after_norm(pending, weight: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """``linear(norm(h + delta), weight)`` for a ``PendingNorm``: in one kernel where that is possible (an
    RMSNorm, bfloat16 weights, at most 16 tokens), otherwise the norm kernel and then the product."""
    from ..parts.norms import RMSNorm

    h, norm = pending.h, pending.norm
    if (isinstance(norm, RMSNorm) and pending.h_new is None and weight.dtype == torch.bfloat16
            and pending.out_dtype == torch.bfloat16 and h.shape[0] <= min(FOLD_NORM_MAX_TOKENS, F.NORMED_MAX_TOKENS) and h.shape[1] % 8 == 0
            and (pending.delta is None or pending.delta.dtype == torch.bfloat16)
            and F.normed_splits(weight.shape[0], h.shape[1]) is not None):
        y, pending.h_new = F.gemm_tc_normed(h, pending.delta, norm.weight, norm.eps, weight, swiglu=swiglu)
        return y
    return linear(pending.materialize(), weight, swiglu=swiglu)


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None,
           swiglu: bool = False) -> torch.Tensor:
    """``x [M, K] @ weight[N, K].T -> [M, N]`` in ``out_dtype`` (default: ``x.dtype``).

    ``swiglu``: ``weight`` holds gate and up rows alternately and the result is ``silu(gate) * up``
    of width ``N / 2``.  ``x`` may be a ``Prescaled`` (rows of an RMSNorm before their division): the
    division is then done where the product is written.
    """
    if isinstance(x, F.Prescaled):
        if weight.dtype == torch.bfloat16 and out_dtype in (None, torch.bfloat16) and weight.data_ptr() % 16 == 0:
            return F.gemm_tc_scaled(x, weight, swiglu=swiglu)
        x = x.materialize()
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
    splits = F.split_k_for(x.shape[0], weight.shape[0], x.shape[1])
    return F.gemm_tc(x, weight, torch.bfloat16 if swiglu else out_dtype, swiglu=swiglu, splits=splits)

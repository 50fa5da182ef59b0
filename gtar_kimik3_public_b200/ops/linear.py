"""The matrix product of a projection, ``y = x @ W.T`` (no bias; src/layers/attention.py:62-65).

The kernel is chosen by the weight's dtype: a float32 weight always goes through the FP32-pipe
kernel (true 32-bit: no tensor cores, no TF32), whatever the activations are; a bfloat16 weight
goes through the kernels of this library with 32-bit accumulation where tokens are few (decode) or an output
stage is fused behind the product (SwiGLU; the q|k|v stage has an entry of its own), and through the library
product, which the reference itself uses for every projection, where many tokens meet a plain product.
"""

from __future__ import annotations

import torch

from . import functional as F
from .library import KernelError, require_device


library_for_plain_products = True  # many-token products without a fused output stage go to the library product
library_from_tokens = F.SKINNY_M    # "many": more tokens than the swap-AB orientation of the own kernel takes

# The library's bfloat16 product must add up in 32-bit throughout, also where it splits K (torch's default lets
# it reduce partial sums in bfloat16); measured, the products here are as fast with the setting off.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


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
    if library_for_plain_products and not swiglu and x.shape[0] > library_from_tokens and out_dtype == torch.bfloat16:
        # many tokens and nothing fused behind the product: the library's product, as in the reference's own
        # engine (nn.Linear, src/engine.py:35).  Measured on a B200 it is 1.1 to 2.7 times as fast as the
        # tensor-memory kernel here on such shapes (it splits K where a product has few tiles and pairs SMs).
        # It writes bfloat16; a product whose result is wanted in 32-bit (the output head) stays on the own kernel,
        # which stores its 32-bit sums, so that logits are the same numbers however many rows a step asks for.
        return F.linear_bf16(x, weight, out_dtype)
    splits = F.split_k_for(x.shape[0], weight.shape[0], x.shape[1])
    return F.gemm_tc(x, weight, torch.bfloat16 if swiglu else out_dtype, swiglu=swiglu, splits=splits)


fold_norms_in_decode = True  # few-token steps: norms inside the products, residual adds in their output stages


def linear_on_stream_ok(h: torch.Tensor, norm_weight: torch.Tensor | None, weight_in: torch.Tensor, weight_out: torch.Tensor) -> bool:
    """Whether a branch ``h += (f(norm(h) @ weight_in.T)) @ weight_out.T`` of a few-token step can run with its norm
    inside the first product (``linear_normed``) and its add inside the last (``linear_residual``)."""
    if not fold_norms_in_decode or norm_weight is None or not h.is_cuda or h.dtype != torch.float32:
        return False
    if weight_in.dtype != torch.bfloat16 or weight_out.dtype != torch.bfloat16 or norm_weight.dtype not in (torch.float32, torch.bfloat16):
        return False
    m = h.shape[0]
    return (m <= F.GEMV_MAX_TOKENS and F.gemv_normed_suits(m, weight_in.shape[0], weight_in.shape[1], h.device)
            and weight_out.shape[1] % 8 == 0 and weight_out.shape[0] % 2 == 0
            and F.gemv_suits(m, weight_out.shape[0], weight_out.shape[1], h.device))


def linear_normed(h: torch.Tensor, norm_weight: torch.Tensor, eps: float, weight: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """``rmsnorm(h; norm_weight, eps) @ weight.T`` (bfloat16) with the norm formed inside the product's kernel."""
    return F.gemv_stream(weight, norm=(h, norm_weight, eps), swiglu=swiglu)


def linear_residual(x: torch.Tensor, weight: torch.Tensor, h: torch.Tensor) -> None:
    """``h += bfloat16(x @ weight.T)`` in the product's output stage."""
    F.gemv_stream(weight, x=x, resid=h)

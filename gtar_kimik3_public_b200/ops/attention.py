"""Attention over the paged cache: picks the kernel for the step's shape and dtype."""

from __future__ import annotations

import torch

from . import functional as F


def paged_attention(q: torch.Tensor, kv: F.PagedKV, ctx, scale: float, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of the step's queries ``[n_tokens, n_q, d]`` over each
    sequence's cached keys and values (the new tokens' own are already written)."""
    return F.attention_exact(q, kv, ctx.tok_pos, ctx.tok_seq, ctx.slots, scale, window)

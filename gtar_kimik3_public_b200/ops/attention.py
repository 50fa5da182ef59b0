"""Attention over the paged cache: picks the kernel for the step's shape and dtype.

* float32, or a head size the tensor-core kernels do not take: the exact kernel (any cut of the
  work gives bit-equal results);
* bfloat16, every sequence bringing one token: the split-KV decode kernel;
* bfloat16 otherwise (prompts, or continuations of several tokens): the flash prefill kernel.
"""

from __future__ import annotations

import os

import torch

from . import functional as F

FAST_HEAD_DIMS = (64, 128)


def fused_decode_ok(qkv: torch.Tensor, kv: F.PagedKV, n_q: int, n_kv: int, head_dim: int) -> bool:
    """Whether the decode kernel that also norms, rotates and writes the new token can take the layer."""
    return (qkv.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16 and head_dim in FAST_HEAD_DIMS
            and kv.page_size == 64 and n_q // n_kv <= 16)


def decode_split_count(ctx, n_kv: int, kv: F.PagedKV) -> int:
    """Blocks that share a sequence's pages in this layer: from the layer's own kv heads and the step's sequence
    lengths (in a captured step the middle of the lengths that the shape's bound covers, not the lengths of the
    day)."""
    sms = F.sm_count(kv.k.device)
    length = ctx.typical_kv_len or ctx.max_kv_len
    return F.decode_splits(ctx.n_seqs, n_kv, length, kv.page_size, sms, F.decode_cluster_places(kv.k.shape[3], sms))


# "auto": the evenly dealt kernel where the estimate favours it; "always" / "never" for measurements
DECODE_FLAT = os.environ.get("GTAR_B200_DECODE_FLAT", "auto")


def decode_flat_preferred(ctx, n_kv: int, kv: F.PagedKV) -> bool:
    """Whether the step's decode attention deals the pages of all sequences out evenly (one kernel, partial
    results through scratch) instead of giving every (sequence, kv head) pair the same number of blocks."""
    if DECODE_FLAT != "auto":
        return DECODE_FLAT == "always"
    sms = F.sm_count(kv.k.device)
    length = ctx.typical_kv_len or ctx.max_kv_len
    return F.decode_flat_wins(ctx.n_seqs, n_kv, length, kv.page_size, sms, F.decode_cluster_places(kv.k.shape[3], sms),
                              F.decode_flat_places(kv.k.shape[3], sms))


def paged_attention(q: torch.Tensor, kv: F.PagedKV, ctx, scale: float, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of the step's queries ``[n_tokens, n_q, d]`` over each
    sequence's cached keys and values (the new tokens' own are already written)."""
    n_q, d = q.shape[1], q.shape[2]
    n_kv = kv.k.shape[1]
    fast = q.dtype == torch.bfloat16 and d in FAST_HEAD_DIMS and kv.page_size == 64 and n_q // n_kv <= 16
    if fast and ctx.all_single:
        if decode_flat_preferred(ctx, n_kv, kv):
            return F.attention_decode_flat(q, None, n_q, n_kv, d, None, None, 1.0, None, None, kv, ctx.kv_len, ctx.slots,
                                           ctx.max_position, scale, window)
        splits = decode_split_count(ctx, n_kv, kv)
        return F.attention_decode(q, kv, ctx.kv_len, ctx.slots, scale, window, splits)
    if fast:
        return F.attention_prefill(q, kv, ctx.cu_q, ctx.kv_len, ctx.slots, ctx.max_q_len, scale, window)
    return F.attention_exact(q, kv, ctx.tok_pos, ctx.tok_seq, ctx.slots, scale, window)

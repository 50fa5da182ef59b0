"""Grouped-query attention with optional per-head q/k RMSNorm and a position encoding.

The reference's ``Attention`` (src/layers/attention.py:49-121): bias-free q/k/v/o projections,
RMSNorm over ``head_dim`` of q and k with one weight each (applied before the rotation),
rotation, cache write, causal attention where consecutive query heads share a kv head, scale
``head_dim ** -0.5``.  Here the three input projections are one packed matrix product, and
norm + rotation + cache write are one kernel.
"""

from __future__ import annotations

import torch

from ..ops import attention as attention_ops
from ..ops import functional as F
from ..ops.linear import linear, linear_normed, linear_on_stream_ok, linear_residual
from .base import KVRequest, Mixer, PositionEncoding, StepContext, TensorSpec, register_part


class GQAAttention(Mixer):
    graph_safe = True  # all per-step numbers are read from device memory by the kernels

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int, qk_norm_eps: float | None,
                 position: PositionEncoding | None, window: int | None = None):
        if n_q_heads % n_kv_heads:
            raise ValueError("query heads must be a multiple of kv heads")
        self.hidden_size, self.n_q, self.n_kv, self.head_dim = int(hidden_size), int(n_q_heads), int(n_kv_heads), int(head_dim)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.position = position
        self.window = window
        self.scale = float(self.head_dim) ** -0.5
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    def tensor_specs(self):
        d, h = self.head_dim, self.hidden_size
        specs = {
            "q_proj.weight": TensorSpec((self.n_q * d, h)),
            "k_proj.weight": TensorSpec((self.n_kv * d, h)),
            "v_proj.weight": TensorSpec((self.n_kv * d, h)),
            "o_proj.weight": TensorSpec((h, self.n_q * d)),
        }
        if self.qk_norm_eps is not None:
            specs["q_norm.weight"] = TensorSpec((d,), "vector")
            specs["k_norm.weight"] = TensorSpec((d,), "vector")
        return specs

    def load(self, tensors):
        parts = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        if len({p.dtype for p in parts}) != 1:  # a file that mixes 32-bit and 16-bit projections
            parts = [p.float() for p in parts]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.qk_norm_eps is not None:
            q_w, k_w = tensors["q_norm.weight"], tensors["k_norm.weight"]
            if q_w.dtype != k_w.dtype:
                q_w, k_w = q_w.float(), k_w.float()
            self.q_norm, self.k_norm = q_w.contiguous(), k_w.contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def cache_request(self):
        return KVRequest(self.n_kv, self.head_dim, self.window)

    def decode_record(self):
        if self.window or self.w_qkv.dtype != torch.bfloat16 or self.w_o.dtype != torch.bfloat16:
            return None
        rope = self.position
        if rope is not None and not (hasattr(rope, "cos") and hasattr(rope, "sin") and getattr(rope, "dim", None) == self.head_dim):
            return None  # another position encoding than tables of cos and sin over the whole head
        return {"kind": "gqa", "hidden": self.hidden_size, "n_q": self.n_q, "n_kv": self.n_kv, "head_dim": self.head_dim,
                "w_qkv": self.w_qkv, "w_o": self.w_o, "q_norm": self.q_norm, "k_norm": self.k_norm,
                "has_qk_norm": self.q_norm is not None, "eps_qk": self.qk_norm_eps or 1.0,
                "qk_dtype": None if self.q_norm is None else self.q_norm.dtype, "rope": rope, "scale": self.scale}

    def forward(self, x, ctx: StepContext, cache: F.PagedKV) -> torch.Tensor:
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.cos, self.position.sin
        write_kv = not ctx.extras.get("cache_read_only", False)
        if F.qkv_fused_ok(x, self.w_qkv, self.head_dim, cache):
            # many tokens: norm, rotation and cache write happen where the projection leaves the tensor cores
            q = F.gemm_tc_qkv(x, self.w_qkv, self.n_q, self.n_kv, self.head_dim, self.q_norm, self.k_norm,
                              self.qk_norm_eps or 1.0, cos, sin, ctx.tok_pos, ctx.tok_seq, ctx.slots, cache,
                              ctx.max_position, write_kv)
            o = attention_ops.paged_attention(q, cache, ctx, self.scale, self.window or 0)
            return linear(o.view(ctx.n_tokens, self.n_q * self.head_dim), self.w_o)
        o = self._attend(linear(x, self.w_qkv), ctx, cache, cos, sin, write_kv)
        return linear(o.view(ctx.n_tokens, self.n_q * self.head_dim), self.w_o)

    def on_stream_ok(self, h: torch.Tensor, norm_weight, ctx: StepContext, cache) -> bool:
        """Whether ``forward_on_stream`` takes this step: a few tokens, one each, bfloat16 matrices of sizes the
        few-token product takes with the norm inside (see ``ops.linear.linear_on_stream_ok``)."""
        return (ctx.all_single and ctx.dtype == torch.bfloat16 and isinstance(cache, F.PagedKV)
                and linear_on_stream_ok(h, norm_weight, self.w_qkv, self.w_o))

    def forward_on_stream(self, h: torch.Tensor, norm_weight: torch.Tensor, norm_eps: float, ctx: StepContext, cache: F.PagedKV) -> None:
        """``h += attention(rmsnorm(h))`` on the 32-bit stream itself: the norm is formed inside the q|k|v product and
        the add happens in the output product's output stage, so the step has two kernels fewer a layer."""
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.cos, self.position.sin
        write_kv = not ctx.extras.get("cache_read_only", False)
        qkv = linear_normed(h, norm_weight, norm_eps, self.w_qkv)
        o = self._attend(qkv, ctx, cache, cos, sin, write_kv)
        linear_residual(o.view(ctx.n_tokens, self.n_q * self.head_dim), self.w_o, h)

    def _attend(self, qkv: torch.Tensor, ctx: StepContext, cache: F.PagedKV, cos, sin, write_kv: bool) -> torch.Tensor:
        """Attention output ``[n_tokens, n_q, head_dim]`` from the packed projection of the step's tokens."""
        if ctx.all_single and attention_ops.fused_decode_ok(qkv, cache, self.n_q, self.n_kv, self.head_dim):
            # one token per sequence: norm, rotation, cache write and attention in one kernel
            if attention_ops.decode_flat_preferred(ctx, self.n_kv, cache):
                return F.attention_decode_flat(
                    None, qkv, self.n_q, self.n_kv, self.head_dim, self.q_norm, self.k_norm, self.qk_norm_eps or 1.0, cos,
                    sin, cache, ctx.kv_len, ctx.slots, ctx.max_position, self.scale, self.window or 0, 0, write_kv)
            splits = attention_ops.decode_split_count(ctx, self.n_kv, cache)
            if splits <= 8:
                return F.attention_decode_fused(
                    qkv, self.n_q, self.n_kv, self.head_dim, self.q_norm, self.k_norm, self.qk_norm_eps or 1.0, cos, sin,
                    cache, ctx.kv_len, ctx.slots, ctx.max_position, self.scale, self.window or 0, splits, write_kv)
        q = F.qk_norm_rope_write(
            qkv, self.n_q, self.n_kv, self.head_dim, self.q_norm, self.k_norm, self.qk_norm_eps or 1.0, cos, sin,
            ctx.tok_pos, ctx.tok_seq, ctx.slots, cache, ctx.max_position, write_kv=write_kv,
        )
        return attention_ops.paged_attention(q, cache, ctx, self.scale, self.window or 0)


register_part("mixer", "gqa_attention", GQAAttention)

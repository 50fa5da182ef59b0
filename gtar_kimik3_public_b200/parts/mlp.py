"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` (src/layers/swiglu.py:9-14), with the gate
and up projections as one packed matrix product whose rows alternate gate, up, gate, up, ... so
that the activation can be applied where the product is written (each output channel's two
numbers sit side by side in the accumulator)."""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.linear import linear, linear_normed, linear_on_stream_ok, linear_residual
from .base import FeedForward, StepContext, TensorSpec, register_part


class SwiGLUFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": TensorSpec((i, h)),
            "up_proj.weight": TensorSpec((i, h)),
            "down_proj.weight": TensorSpec((h, i)),
        }

    def load(self, tensors):
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def decode_record(self):
        if self.w_gate_up.dtype != torch.bfloat16 or self.w_down.dtype != torch.bfloat16:
            return None
        return {"kind": "swiglu", "hidden": self.hidden_size, "inter": self.intermediate_size, "w_gu": self.w_gate_up,
                "w_down": self.w_down}

    def forward(self, x, ctx: StepContext) -> torch.Tensor:
        return linear(linear(x, self.w_gate_up, swiglu=True), self.w_down)

    def on_stream_ok(self, h: torch.Tensor, norm_weight, ctx: StepContext) -> bool:
        return ctx.dtype == torch.bfloat16 and linear_on_stream_ok(h, norm_weight, self.w_gate_up, self.w_down)

    def forward_on_stream(self, h: torch.Tensor, norm_weight: torch.Tensor, norm_eps: float, ctx: StepContext) -> None:
        """``h += down(silu(gate(y)) * up(y))`` with ``y = rmsnorm(h)`` formed inside the gate|up product and the add
        in the down product's output stage."""
        linear_residual(linear_normed(h, norm_weight, norm_eps, self.w_gate_up, swiglu=True), self.w_down, h)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)

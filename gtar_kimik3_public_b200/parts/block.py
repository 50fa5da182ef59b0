"""Pre-norm residual block: ``h += mixer(norm_in(h)); h += ffn(norm_post(h))``
(src/models/transformer.py:47-48).  The adds are fused into the norm that follows them: the
block hands its last branch output on as ``pending`` instead of adding it itself."""

from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm, StepContext, register_part


class PreNormBlock(Block):
    def __init__(self, input_norm: Norm, mixer: Mixer, post_norm: Norm, feed_forward: FeedForward,
                 names: dict[str, str] | None = None):
        self.input_norm, self.mixer, self.post_norm, self.feed_forward = input_norm, mixer, post_norm, feed_forward
        # tensor-name prefixes of the four parts inside the layer
        self.names = names or {
            "input_norm": "input_layernorm.",
            "mixer": "self_attn.",
            "post_norm": "post_attention_layernorm.",
            "feed_forward": "mlp.",
        }

    def children(self):
        return [(self.names[k], getattr(self, k)) for k in ("input_norm", "mixer", "post_norm", "feed_forward")]

    def tensor_specs(self):
        return {prefix + name: spec for prefix, part in self.children() for name, spec in part.tensor_specs().items()}

    def load(self, tensors):
        for prefix, part in self.children():
            part.load({name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)})

    def weight_bytes(self):
        return sum(part.weight_bytes() for _, part in self.children())

    def forward(self, h, pending, ctx: StepContext, cache):
        x = self.input_norm.forward(h, pending, ctx.dtype)
        branch = self.mixer.forward(x, ctx, cache)
        x = self.post_norm.forward(h, branch, ctx.dtype)
        return h, self.feed_forward.forward(x, ctx)


register_part("block", "pre_norm", PreNormBlock)

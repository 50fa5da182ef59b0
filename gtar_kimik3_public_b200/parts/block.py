"""Pre-norm residual block: ``h += mixer(norm_in(h)); h += ffn(norm_post(h))``
(src/models/transformer.py:47-48).  The adds are fused into the norm that follows them: the
block hands its last branch output on as ``pending`` instead of adding it itself."""

from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm, PendingNorm, StepContext, register_part, resolve


class PreNormBlock(Block):
    takes_deferred = True  # ``pending`` may be a DeferredProjection

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
        # a part that can leaves its last projection to the norm after it (of this layer or the next)
        x = self._normed(self.input_norm, h, pending, ctx, self.mixer)
        if getattr(self.mixer, "can_defer_output", False) and getattr(self.post_norm, "takes_deferred", False):
            branch = self.mixer.forward(x, ctx, cache, defer=True)
        else:
            branch = self.mixer.forward(x, ctx, cache)
        h = x.stream() if isinstance(x, PendingNorm) else h
        x = self._normed(self.post_norm, h, branch, ctx, self.feed_forward)
        if getattr(self.feed_forward, "can_defer_output", False):
            out = self.feed_forward.forward(x, ctx, defer=True)
        else:
            out = self.feed_forward.forward(x, ctx)
        h = x.stream() if isinstance(x, PendingNorm) else h
        return h, out

    @staticmethod
    def _normed(norm: Norm, h, delta, ctx: StepContext, consumer):
        """The consumer's input: normalised activations, or, where norm and consumer can, rows that the
        consumer's first projection still has to divide by their root mean square."""
        if getattr(norm, "takes_deferred", False):
            return norm.forward(h, delta, ctx.dtype, prescaled_ok=getattr(consumer, "accepts_prescaled", False))
        delta = resolve(delta)
        if getattr(consumer, "accepts_pending_norm", False):
            return PendingNorm(h, delta, norm, ctx.dtype)
        return norm.forward(h, delta, ctx.dtype)


register_part("block", "pre_norm", PreNormBlock)

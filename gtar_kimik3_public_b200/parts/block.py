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

    def decode_record(self) -> dict | None:
        """What the persistent decode kernel needs of this layer (weights, constants, sizes), or None when one of
        the four parts is not of the kind that kernel computes; each part answers for itself."""
        pieces = {}
        for key, part in (("in", self.input_norm), ("mixer", self.mixer), ("post", self.post_norm), ("ffn", self.feed_forward)):
            describe = getattr(part, "decode_record", None)
            piece = describe() if describe is not None else None
            if piece is None:
                return None
            pieces[key] = piece
        norm_in, norm_post, mixer, ffn = pieces["in"], pieces["post"], pieces["mixer"], pieces["ffn"]
        if mixer.get("kind") != "gqa" or ffn.get("kind") != "swiglu" or norm_in.get("kind") != "rmsnorm" or norm_post.get("kind") != "rmsnorm":
            return None
        if not (norm_in["size"] == norm_post["size"] == mixer["hidden"] == ffn["hidden"]):
            return None
        if norm_in["weight"].dtype != norm_post["weight"].dtype:
            return None
        return {**mixer, "inter": ffn["inter"], "w_gu": ffn["w_gu"], "w_down": ffn["w_down"], "norm_in": norm_in["weight"],
                "norm_post": norm_post["weight"], "eps_in": norm_in["eps"], "eps_post": norm_post["eps"],
                "norm_dtype": norm_in["weight"].dtype}

    @staticmethod
    def _plain_rmsnorm(norm):
        """(weight, eps) of a norm that is nothing but an RMSNorm with a weight, else None."""
        describe = getattr(norm, "decode_record", None)
        record = describe() if describe is not None else None
        return (record["weight"], record["eps"]) if record and record.get("kind") == "rmsnorm" else None

    def forward(self, h, pending, ctx: StepContext, cache):
        # Few-token steps: a branch may work on the stream itself (``forward_on_stream``: its norm inside its first
        # product, its add inside its last), which saves the two norm kernels of the layer.  A part that offers no such
        # method, a norm of another kind or sizes the kernels do not take leave the branch as it is below.
        if pending is None and ctx.n_tokens <= 16:
            norm = self._plain_rmsnorm(self.input_norm)
            ok = getattr(self.mixer, "on_stream_ok", None)
            if norm is not None and ok is not None and ok(h, norm[0], ctx, cache):
                self.mixer.forward_on_stream(h, norm[0], norm[1], ctx, cache)
                norm = self._plain_rmsnorm(self.post_norm)
                ok = getattr(self.feed_forward, "on_stream_ok", None)
                if norm is not None and ok is not None and ok(h, norm[0], ctx):
                    self.feed_forward.forward_on_stream(h, norm[0], norm[1], ctx)
                    return h, None
                x = self.post_norm.forward(h, None, ctx.dtype)
                return h, self.feed_forward.forward(x, ctx)
        x = self.input_norm.forward(h, pending, ctx.dtype)
        branch = self.mixer.forward(x, ctx, cache)
        x = self.post_norm.forward(h, branch, ctx.dtype)
        return h, self.feed_forward.forward(x, ctx)


register_part("block", "pre_norm", PreNormBlock)

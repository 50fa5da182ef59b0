"""The Qwen3-style dense decoder (arch ``"transformer"``) put together from parts.

The reference's stack (src/models/transformer.py:27-67,70-77): token embedding; per layer a
pre-norm block of GQA attention (per-head q/k RMSNorm, rotary positions over the whole head)
and a SwiGLU feed-forward; a final RMSNorm; an output head that may be tied to the embedding.
Every layer is alike and the layers run once each in order, so the run list is ``0..L-1``.
"""

from __future__ import annotations

from ..config.transformer import TransformerConfig
from ..parts.base import build_part
from ..parts.embedding import OutputHead, TokenEmbedding
from .model import ModelPlan, RunEntry


def build_transformer_plan(config: TransformerConfig) -> ModelPlan:
    rope = build_part("position", "rope", dim=config.head_dim, base=config.rope_theta)
    layers = []
    for _ in range(config.num_hidden_layers):
        mixer = build_part(
            "mixer", "gqa_attention", hidden_size=config.hidden_size, n_q_heads=config.num_attention_heads,
            n_kv_heads=config.num_key_value_heads, head_dim=config.head_dim, qk_norm_eps=config.rms_norm_eps,
            position=rope,
        )
        ffn = build_part("feed_forward", "swiglu", hidden_size=config.hidden_size,
                         intermediate_size=config.intermediate_size)
        layers.append(build_part(
            "block", "pre_norm",
            input_norm=build_part("norm", "rmsnorm", size=config.hidden_size, eps=config.rms_norm_eps),
            mixer=mixer,
            post_norm=build_part("norm", "rmsnorm", size=config.hidden_size, eps=config.rms_norm_eps),
            feed_forward=ffn,
        ))
    embedding = TokenEmbedding(config.vocab_size, config.hidden_size)
    head = OutputHead(config.hidden_size, config.vocab_size, tied_to=embedding if config.tie_word_embeddings else None)
    return ModelPlan(
        embedding=embedding,
        layers=layers,
        final_norm=build_part("norm", "rmsnorm", size=config.hidden_size, eps=config.rms_norm_eps),
        head=head,
        run_list=[RunEntry(i) for i in range(config.num_hidden_layers)],
        positions=[rope],
    )

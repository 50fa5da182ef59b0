"""Configuration of the Qwen3-style dense decoder (arch ``"transformer"``).

Field names are the reference's (``src/models/transformer.py:12-24``); the same names are
what a Qwen3 model folder's config.json uses.  ``vocab_size`` is not in the reference's
JSON files (its callers inject it, ``scripts/train.py:83-85``), so a model folder written
by this library always carries it.
"""

from __future__ import annotations

import dataclasses
from typing import ClassVar

from .base import ConfigError, ModelConfig


@dataclasses.dataclass(frozen=True)
class TransformerConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    # Optional keys: they do not change the function the model computes.
    initializer_range: float | None = None  # only read by the random-weights mode
    max_position_embeddings: int | None = None  # longest sequence a request may reach
    eos_token_id: int | None = None
    bos_token_id: int | None = None
    pad_token_id: int | None = None

    ARCH_NAMES: ClassVar[tuple[str, ...]] = ("transformer", "Qwen3ForCausalLM")
    IGNORED_KEYS: ClassVar[frozenset[str]] = frozenset(
        {"torch_dtype", "dtype", "transformers_version", "use_cache", "max_window_layers", "sliding_window"}
    )
    # The reference's block has exactly one shape: SiLU gate, no biases, no dropout, full
    # rotary, no window (src/layers/attention.py:62-67, src/layers/swiglu.py:9-14).
    FIXED_KEYS: ClassVar[dict] = {
        "hidden_act": ("silu",),
        "attention_bias": (False,),
        "attention_dropout": (0, 0.0),
        "use_sliding_window": (False,),
        "rope_scaling": (None,),
        "mlp_bias": (False,),
    }

    def validate(self) -> None:
        for name in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
        ):
            if getattr(self, name) <= 0:
                raise ConfigError(f"TransformerConfig: {name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"TransformerConfig: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 8 != 0:
            raise ConfigError(f"TransformerConfig: head_dim ({self.head_dim}) must be a multiple of 8 (the attention "
                              "kernels read a head's row in 16- or 32-byte pieces; rotary pairs need it even)")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"TransformerConfig: rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"TransformerConfig: rope_theta must be > 0, got {self.rope_theta}")
        if self.max_position_embeddings is not None and self.max_position_embeddings <= 0:
            raise ConfigError("TransformerConfig: max_position_embeddings must be positive")
        for name in ("eos_token_id", "bos_token_id", "pad_token_id"):
            value = getattr(self, name)
            if value is not None and not (0 <= value < self.vocab_size):
                raise ConfigError(f"TransformerConfig: {name} ({value}) is outside the vocabulary")

"""Typed configurations."""

from .base import ConfigError, ModelConfig, architecture_name, read_config_json  # noqa: F401
from .transformer import TransformerConfig  # noqa: F401

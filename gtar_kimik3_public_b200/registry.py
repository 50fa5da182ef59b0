"""One registry from an architecture's name to its configuration class and model builder.

The reference's is ``ARCHITECTURES[arch] -> (Config, ForCausalLM)`` (src/models/__init__.py:5-8),
looked up with the config file's ``"arch"`` (scripts/generate.py:32).  The same lookup is used
everywhere here: the loader, the command line, trace replay and the benchmark.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .config.base import ConfigError, ModelConfig, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type[ModelConfig]
    build_plan: Callable  # config -> ModelPlan


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(names, config_class: type[ModelConfig], build_plan: Callable, replace: bool = False) -> None:
    for name in names:
        if name in _ARCHITECTURES and not replace:
            raise KeyError(f"architecture {name!r} is already registered")
        _ARCHITECTURES[name] = Architecture(name, config_class, build_plan)


def architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; known: {sorted(_ARCHITECTURES)}") from None


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def config_from_dict(raw: dict) -> ModelConfig:
    return architecture(architecture_name(raw)).config_class.from_dict(raw)


def config_from_file(path, overrides: dict | None = None) -> ModelConfig:
    """Reads a model folder's config.json (or the reference's nested training config); ``overrides``
    supplies keys such a file lacks (the reference's files carry no ``vocab_size``)."""
    raw = read_config_json(path)
    if overrides:
        raw = {**raw, **overrides}
    return config_from_dict(raw)


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from .config.transformer import TransformerConfig
    from .models.transformer import build_transformer_plan

    register_architecture(TransformerConfig.ARCH_NAMES, TransformerConfig, build_transformer_plan)

"""Typed model configuration: the common machinery every architecture's config shares.

A configuration class is a frozen dataclass whose field names are the keys of the
architecture's own ``config.json``.  Fields without a default are required keys; nothing
that the file gives is replaced by a constant in code.  The reference builds its config
the same way, straight from the JSON's keys (``src/models/transformer.py:12-24``,
``scripts/generate.py:32-36``), except that it carries class defaults; here a model
folder has to say every size itself.
"""

from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the chosen architecture."""


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configurations.

    Subclasses list their keys as dataclass fields, name the architecture strings they
    answer to in ``ARCH_NAMES`` and check relations between fields in ``validate``.
    ``IGNORED_KEYS`` are keys commonly found in model folders that carry no information
    for inference; ``FIXED_KEYS`` maps keys that this architecture does not vary to the
    only value it accepts (a file that says otherwise is refused, never silently
    reinterpreted).
    """

    ARCH_NAMES: ClassVar[tuple[str, ...]] = ()
    IGNORED_KEYS: ClassVar[frozenset[str]] = frozenset()
    FIXED_KEYS: ClassVar[dict[str, tuple[Any, ...]]] = {}

    @classmethod
    def field_names(cls) -> list[str]:
        return [f.name for f in dataclasses.fields(cls)]

    @classmethod
    def required_keys(cls) -> list[str]:
        return [
            f.name
            for f in dataclasses.fields(cls)
            if f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING
        ]

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        known = set(cls.field_names())
        values: dict[str, Any] = {}
        unknown: list[str] = []
        for key, value in raw.items():
            if key in known:
                values[key] = value
            elif key in cls.FIXED_KEYS:
                if value not in cls.FIXED_KEYS[key]:
                    raise ConfigError(
                        f"{cls.__name__}: key {key!r} = {value!r} is not supported by this "
                        f"architecture (accepted: {list(cls.FIXED_KEYS[key])})"
                    )
            elif key in cls.IGNORED_KEYS or key in ("arch", "architectures", "model_type"):
                continue
            else:
                unknown.append(key)
        missing = [k for k in cls.required_keys() if k not in values]
        if missing or unknown:
            parts = []
            if missing:
                parts.append(f"missing keys {sorted(missing)}")
            if unknown:
                parts.append(f"unknown keys {sorted(unknown)}")
            raise ConfigError(f"{cls.__name__}: " + "; ".join(parts))
        config = cls(**cls._coerce(values))
        config.validate()
        return config

    @classmethod
    def _coerce(cls, values: dict[str, Any]) -> dict[str, Any]:
        """Bring JSON values to the field's type (ints stay ints, 1e6 becomes a float)."""
        out = {}
        types = {f.name: f.type for f in dataclasses.fields(cls)}
        for key, value in values.items():
            kind = str(types[key])
            if value is None:
                out[key] = None
            elif kind.startswith("int"):
                if isinstance(value, bool) or int(value) != value:
                    raise ConfigError(f"{cls.__name__}: key {key!r} must be an integer, got {value!r}")
                out[key] = int(value)
            elif kind.startswith("float"):
                if isinstance(value, bool):
                    raise ConfigError(f"{cls.__name__}: key {key!r} must be a number, got {value!r}")
                out[key] = float(value)
            elif kind.startswith("bool"):
                if not isinstance(value, bool):
                    raise ConfigError(f"{cls.__name__}: key {key!r} must be true or false, got {value!r}")
                out[key] = value
            else:
                out[key] = value
        return out

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    def to_dict(self) -> dict[str, Any]:
        out = dataclasses.asdict(self)
        if self.ARCH_NAMES:
            out["arch"] = self.ARCH_NAMES[0]
        return out


def read_config_json(path: str | Path) -> dict[str, Any]:
    """Read a config file and flatten the two layouts that exist.

    A model folder's ``config.json`` is flat.  The reference's training configs are
    nested, ``{"arch": ..., "model": {...}, "train": {...}}`` (``configs/transformer_0.6B.json``);
    their ``model`` section is lifted to the top level and ``train`` is dropped.
    """
    path = Path(path)
    if path.is_dir():
        path = path / "config.json"
    try:
        raw = json.loads(path.read_text())
    except FileNotFoundError:
        raise ConfigError(f"no config file at {path}") from None
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    if isinstance(raw.get("model"), dict):
        flat = dict(raw["model"])
        for key, value in raw.items():
            if key not in ("model", "train"):
                flat[key] = value
        raw = flat
    return raw


def architecture_name(raw: dict[str, Any]) -> str:
    """The architecture string of a config dict: ``arch`` or the first of ``architectures``."""
    if isinstance(raw.get("arch"), str):
        return raw["arch"]
    names = raw.get("architectures")
    if isinstance(names, (list, tuple)) and names and isinstance(names[0], str):
        return names[0]
    raise ConfigError('config has neither "arch" nor "architectures"; cannot choose a model class')

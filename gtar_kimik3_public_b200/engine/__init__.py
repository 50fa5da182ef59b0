"""The step function and the generation loop."""

from .engine import Engine, StepEntry  # noqa: F401

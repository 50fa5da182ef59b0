"""The generic model and the architectures built on it."""

from .model import Model, ModelPlan, RunEntry  # noqa: F401

"""Greedy and temperature (+ top-k) sampling."""

from .sampler import SamplingParams, choose  # noqa: F401

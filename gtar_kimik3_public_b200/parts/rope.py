"""Rotary position encoding: tables of cos and sin of ``position * inv_freq``.

``inv_freq[i] = 1 / base^(2i/dim)`` is built in float32 by the reference's own expression and
the angle is a float32 product (src/layers/rope.py:8,11-14); the rotation pairs element ``i``
with ``i + dim/2`` (rope.py:17-19).  The tables hold the ``dim/2`` distinct angles per position
and are made on the device once, for as many positions as the cache can hold.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, dim: int, base: float):
        if dim % 2:
            raise ValueError(f"rotary dimension must be even, got {dim}")
        self.dim = int(dim)
        self.base = float(base)
        self.cos: torch.Tensor | None = None
        self.sin: torch.Tensor | None = None
        self._replaced: list[torch.Tensor] = []  # shorter tables of before: captured launches may still read them

    def inv_freq(self) -> torch.Tensor:
        return 1.0 / (self.base ** (torch.arange(0, self.dim, 2, dtype=torch.float32) / self.dim))

    def prepare(self, max_position: int, device: torch.device) -> None:
        have = 0 if self.cos is None else self.cos.shape[0]
        if self.cos is not None and self.cos.device == device and have > max_position:
            return
        if self.cos is not None:
            # A CUDA graph captured earlier holds the old tables' addresses.  Their rows stay right (a row depends
            # on its position only), so they are kept instead of freed.
            self._replaced += [self.cos, self.sin]
        n = max(max_position + 1, 2 * have, 64)
        positions = torch.arange(n, dtype=torch.float32, device=device)
        freqs = positions[:, None] * self.inv_freq().to(device)[None, :]
        self.cos = freqs.cos().contiguous()
        self.sin = freqs.sin().contiguous()


register_part("position", "rope", RotaryEncoding)

"""The interfaces of the parts a model is put together from, and the registries that name them.

A model is a list of layers; a layer is a *block* that arranges a *mixer* (attention here), a
*feed-forward* and *norms* around the residual stream; mixers may use a *position encoding*.
Each part is built from numbers (its sizes and constants) — never from a config object and
never knowing which model it sits in, as the reference's layers are
(``Attention(hidden, nq, nkv, d, eps)``, ``SwiGLU(hidden, inter)``, ``RMSNorm(n, eps)``,
``RotaryEmbedding(dim, base)``; src/models/transformer.py:30-39,58).

What a part must offer:

* ``tensor_specs()``: the tensors it reads from a model folder, by name relative to the part,
  with their shapes — the loader checks the file against these before any device work;
* ``load(tensors)``: takes those tensors (already on the device, in the dtype the loader's rule
  gives) and may repack them;
* ``forward(...)``: runs on the packed activations of one step.

Mixers also say what they need kept between steps (``cache_request()``): keys and values for
every position, for a window of positions, a state of fixed size, several of these, or nothing.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class TensorSpec:
    """Shape and kind of one named tensor.  Kinds: ``matrix``/``vector`` (floating point, kept in
    bfloat16 unless the file stores 32-bit), ``table`` (integers, kept as int32)."""

    shape: tuple[int, ...]
    kind: str = "matrix"
    optional: bool = False


@dataclass(frozen=True)
class KVRequest:
    """Keys and values per position.  ``window`` = None keeps all positions."""

    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateRequest:
    """A per-sequence state of fixed size (does not grow with the sequence), zero at the start."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class StepContext:
    """What every part may know about the step being run.  All tensors are on the device.

    The step holds ``n_seqs`` sequences; sequence ``i`` brings ``q_len[i]`` new tokens after
    ``past_len[i]`` cached ones.  Tokens are packed in sequence order.
    """

    n_tokens: int
    n_seqs: int
    dtype: torch.dtype  # activation dtype of this run: bfloat16 or float32
    tokens: torch.Tensor  # [n_tokens] int32
    tok_pos: torch.Tensor  # [n_tokens] int32, position of each token in its sequence
    tok_seq: torch.Tensor  # [n_tokens] int32, index (0..n_seqs-1) of each token's sequence
    cu_q: torch.Tensor  # [n_seqs + 1] int32, start of each sequence's tokens
    slots: torch.Tensor  # [n_seqs] int32, cache slot of each sequence
    kv_len: torch.Tensor  # [n_seqs] int32, tokens cached after this step (past + new)
    want_rows: torch.Tensor  # [n_want] int32, packed token rows whose logits are asked for
    max_q_len: int  # host copies of what kernels need to size their launches
    max_kv_len: int
    max_position: int
    all_single: bool  # every sequence brings exactly one token (a decode step)
    # where max_kv_len is a bound for many steps to come and not the longest length of this one: a length in the
    # middle of what the bound covers, to choose launch shapes by (0: there is none, max_kv_len is the length)
    typical_kv_len: int = 0
    host_q_len: list[int] = field(default_factory=list)
    host_past_len: list[int] = field(default_factory=list)
    host_slots: list[int] = field(default_factory=list)
    extras: dict[str, Any] = field(default_factory=dict)


class Part:
    """Common face of every part."""

    # Whether the part's forward() may be captured in a CUDA graph: it launches kernels only, and every
    # number that changes from step to step is read from device memory.  A part that looks at host copies
    # of lengths, loops over sequences on the host or waits for the device says False (the default), and a
    # model with such a part runs its steps launch by launch.
    graph_safe = False

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no tensors")

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads from this part (for roofline accounting)."""
        return 0


class Norm(Part):
    def forward(self, h: torch.Tensor, delta: torch.Tensor | None, out_dtype: torch.dtype,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        """Adds ``delta`` into the 32-bit stream ``h`` (in place) and returns the normalised rows."""
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, max_position: int, device: torch.device) -> None:
        """Makes sure positions ``0..max_position`` can be encoded (tables grown before a step)."""


class Mixer(Part):

    def cache_request(self) -> KVRequest | StateRequest | None | list:
        """What the mixer needs kept between steps: a ``KVRequest``, a ``StateRequest``, None, or a list of
        requests (keys and values and a state; several state tensors of their own shapes and types).  ``forward``
        gets the storage in the same form: one view, None, or a tuple of views in the list's order."""
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Any) -> torch.Tensor:
        """``x``: normalised activations ``[n_tokens, hidden]``; returns the branch output, same shape."""
        raise NotImplementedError


class FeedForward(Part):

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of the parts of one layer around the residual stream."""

    def children(self) -> list[tuple[str, Part]]:
        """(tensor-name prefix, part) of everything inside the block."""
        return []

    @property
    def graph_safe(self) -> bool:
        parts = self.children()
        return bool(parts) and all(part.graph_safe for _, part in parts)

    mixer: Mixer

    def forward(self, h: torch.Tensor, pending: torch.Tensor | None, ctx: StepContext,
                cache: Any) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Runs the layer.  ``h`` is the 32-bit residual stream, ``pending`` a branch output not yet
        added to it (so that the add can be fused with the next norm).  Returns the stream (the same
        tensor updated in place, or a new one) and the new pending."""
        raise NotImplementedError


# ------------------------------------------------------------------ registries of part kinds
_REGISTRIES: dict[str, dict[str, Callable[..., Part]]] = {
    "mixer": {},
    "feed_forward": {},
    "norm": {},
    "position": {},
    "block": {},
}


def register_part(family: str, name: str, factory: Callable[..., Part], replace: bool = False) -> None:
    """Makes ``factory(**params)`` available under ``name`` in one of the families
    ``mixer``, ``feed_forward``, ``norm``, ``position``, ``block``."""
    if family not in _REGISTRIES:
        raise KeyError(f"unknown part family {family!r}; families are {sorted(_REGISTRIES)}")
    if name in _REGISTRIES[family] and not replace:
        raise KeyError(f"{family} {name!r} is already registered")
    _REGISTRIES[family][name] = factory


def build_part(family: str, name: str, **params) -> Part:
    try:
        factory = _REGISTRIES[family][name]
    except KeyError:
        raise KeyError(f"no {family} named {name!r}; known: {sorted(_REGISTRIES.get(family, {}))}") from None
    return factory(**params)


def known_parts(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])

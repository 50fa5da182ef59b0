"""The generic model: an embedding, a list of layers, a run list, a final norm and a head.

Nothing here knows an architecture.  An architecture's builder (for instance
``models/transformer.py``) turns its configuration into a ``ModelPlan``: the parts, the tensor
name prefix of each, and the order in which layers run.  The run list is data: it may name a
layer twice (the layer's weights are then used twice, each run with storage of its own) or let
an entry read the storage that an earlier entry writes.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..cache import Cache, CacheLayout
from ..ops import functional as F
from ..parts.base import Block, Norm, Part, PositionEncoding, StepContext, TensorSpec
from ..parts.embedding import OutputHead, TokenEmbedding


@dataclass
class RunEntry:
    """One step of the run list: which layer runs, and whose storage it uses (None: its own)."""

    layer: int
    cache_of: int | None = None  # index of an earlier run-list entry


@dataclass
class ModelPlan:
    embedding: TokenEmbedding
    layers: list[Block]
    final_norm: Norm
    head: OutputHead
    run_list: list[RunEntry]
    positions: list[PositionEncoding] = field(default_factory=list)
    embedding_prefix: str = "model.embed_tokens."
    layer_prefix: str = "model.layers.{}."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."


class Model:
    def __init__(self, plan: ModelPlan, config, dtype: torch.dtype, device: torch.device | str):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"a model runs in float32 or bfloat16, not {dtype}")
        self.plan, self.config, self.dtype, self.device = plan, config, dtype, torch.device(device)
        for position, entry in enumerate(plan.run_list):
            if not 0 <= entry.layer < len(plan.layers):
                raise ValueError(f"run-list entry {position} names layer {entry.layer}; there are {len(plan.layers)}")
            if entry.cache_of is not None and not 0 <= entry.cache_of < position:
                raise ValueError(f"run-list entry {position} may only read the storage of an earlier entry")
        self.vocab_size = plan.head.vocab_size

    # ------------------------------------------------------------------ weights
    def named_parts(self) -> list[tuple[str, Part]]:
        plan = self.plan
        parts: list[tuple[str, Part]] = [(plan.embedding_prefix, plan.embedding)]
        parts += [(plan.layer_prefix.format(i), layer) for i, layer in enumerate(plan.layers)]
        parts += [(plan.final_norm_prefix, plan.final_norm), (plan.head_prefix, plan.head)]
        return parts

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {prefix + name: spec for prefix, part in self.named_parts() for name, spec in part.tensor_specs().items()}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for prefix, part in self.named_parts():
            part.load({name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)})

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one decode step reads: every run-list entry's layer, the final norm and
        the head (the embedding contributes single rows and is left out)."""
        plan = self.plan
        total = sum(plan.layers[e.layer].weight_bytes() for e in plan.run_list)
        return total + plan.final_norm.weight_bytes() + plan.head.weight_bytes()

    # ------------------------------------------------------------------ cache
    def cache_layout(self) -> CacheLayout:
        plan = self.plan
        requests = [plan.layers[e.layer].mixer.cache_request() for e in plan.run_list]
        shared = {i: e.cache_of for i, e in enumerate(plan.run_list) if e.cache_of is not None}
        return CacheLayout(requests, shared)

    def make_cache(self, max_tokens: int, max_seqs: int | None = None) -> Cache:
        max_len = getattr(self.config, "max_position_embeddings", None)
        return Cache(self.cache_layout(), max_tokens, self.dtype, self.device, max_seqs=max_seqs, max_seq_len=max_len)

    def graph_safe(self) -> bool:
        """Whether a decode step may be captured in a CUDA graph: every part of the plan must say so (a part
        that does host work per step, as test fixtures may, keeps the step out of graphs)."""
        plan = self.plan
        parts = [plan.embedding, plan.final_norm, plan.head, *plan.positions, *(plan.layers[e.layer] for e in plan.run_list)]
        return all(getattr(part, "graph_safe", False) for part in parts)

    def persistent_decode(self, cache: Cache):
        """The plan that runs all layers of a small decode step as one kernel on this cache (made once per cache),
        or None if the model's layers, its sizes or the cache are not what that kernel takes."""
        plans = self.__dict__.setdefault("_persistent_plans", {})
        key = id(cache)
        if key not in plans or plans[key][0]() is not cache:
            import weakref

            from .persistent_decode import build

            plans[key] = (weakref.ref(cache), build(self, cache))
        return plans[key][1]

    # ------------------------------------------------------------------ the forward pass of one step
    def prepare(self, max_position: int) -> None:
        for position in self.plan.positions:
            position.prepare(max_position, self.device)

    def step(self, ctx: StepContext, cache: Cache) -> torch.Tensor:
        """Runs the step's tokens through the run list and returns float32 logits ``[n_want, vocab]``
        at ``ctx.want_rows``."""
        plan = self.plan
        self.prepare(ctx.max_position)
        h = plan.embedding.forward(ctx.tokens)
        pending = None
        persistent = self.persistent_decode(cache) if ctx.all_single and ctx.n_seqs <= F.DECODE_LAYERS_MAX_SEQS else None
        if persistent is not None:
            persistent.run(h, ctx)  # every layer of the run list in one kernel; the stream is complete afterwards
        else:
            for index, entry in enumerate(plan.run_list):
                ctx.extras["cache_read_only"] = cache.is_shared(index)
                h, pending = plan.layers[entry.layer].forward(h, pending, ctx, cache.view(index))
        if ctx.want_rows.numel() == 0:
            # nothing asked for: still fold the last branch into the stream so the step is whole
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        z = plan.final_norm.forward(h, pending, ctx.dtype, rows=ctx.want_rows)
        return plan.head.forward(z)

"""Steps replayed from CUDA graphs.

A step launches some hundred kernels; issued one by one from Python they cost more host time
than device time for all but the longest prompts.  A step's launches depend only on its *shape*
— how many tokens, sequences and wanted rows, the longest sequence part — while everything else
(token ids, positions, slots, lengths, the page table) lives in device memory that the kernels
read.  So the whole step, embedding to logits, is captured once per shape and replayed; the
host's work per step is one small pinned copy of those numbers.  Decode steps (one token per
sequence) are captured at their first use, other shapes when they are seen a second time; the
least recently used graphs are dropped beyond a limit.

A decode shape also carries a bound on the longest sequence of the step (``MIN_LENGTH_BOUND`` times a
power of two or one and a half times that: 1,024, 1,536, 2,048, 3,072, ..., at most what the cache holds):
kernels size their launches from that bound, not from the lengths of the day, so a short context in a
cache made for long ones is not cut into as many pieces as the longest context would need.  Where a
launch shape is a matter of speed only (into how many blocks a sequence's pages are cut), it is chosen
for the middle of the lengths that the bound covers.

A step is executed exactly once, also the step at which its shape is captured: that step runs launch
by launch (which does whatever one-time set-up the kernels need) and gives the result, the capture
after it executes nothing, and replays serve the later steps.  A part that advances a state in place
may therefore be graph-safe.

Inside a graph every kernel is launched with programmatic stream serialization: it may start
(and fetch weights) while the kernel before it drains, and waits for that kernel's results only
where it first needs them.
"""

from __future__ import annotations

from collections import OrderedDict

import numpy as np
import torch

from ..ops.functional import set_pdl
from .step import PackedStep, context_from_views


class StepGraphs:
    RING = 8
    MAX_PREFILL_GRAPHS = 12
    MIN_LENGTH_BOUND = 1024

    def __init__(self, model, cache, use_pdl: bool = True):
        self.model, self.cache, self.use_pdl = model, cache, use_pdl
        device = model.device
        self.t_max = cache.n_pages * cache.page_size  # no step can bring more tokens than the cache holds
        self.s_max = cache.max_seqs
        # tokens | positions | sequence of token | starts | slots | lengths | wanted rows, one after
        # another from the front of the buffer: for a given shape every field has a fixed address
        total = 4 * self.t_max + 3 * self.s_max + 1
        self.meta = torch.zeros(total, dtype=torch.int32, device=device)
        self.host = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.host_np = [h.numpy() for h in self.host]
        self.events: list[torch.cuda.Event | None] = [None] * self.RING
        self.turn = 0
        self.graphs: OrderedDict[tuple, tuple[torch.cuda.CUDAGraph, torch.Tensor]] = OrderedDict()
        self.seen: set[tuple] = set()
        self.pool = None
        self.launches: dict[tuple, int] = {}

    # ------------------------------------------------------------------ step inputs
    @staticmethod
    def offsets(packed: PackedStep) -> list[int]:
        out, at = [], 0
        for field in packed.fields:
            out.append(at)
            at += len(field)
        return out + [at]

    def views(self, packed: PackedStep) -> list[torch.Tensor]:
        offsets = self.offsets(packed)
        return [self.meta[o:o + len(f)] for o, f in zip(offsets, packed.fields)]

    def upload(self, packed: PackedStep, skip_tokens: bool) -> None:
        """Puts the step's numbers where the captured kernels read them.  The pinned buffers are
        used in turn, each guarded by an event, so that a copy still waiting in the stream is never
        overwritten by the host."""
        turn = self.turn
        self.turn = (turn + 1) % self.RING
        if self.events[turn] is not None:
            self.events[turn].synchronize()
        buf, pinned = self.host_np[turn], self.host[turn]
        offsets = self.offsets(packed)
        for offset, field in zip(offsets, packed.fields):
            buf[offset:offset + len(field)] = field
        begin = offsets[1] if skip_tokens else 0  # the token ids come from the device in that case
        self.meta[begin:offsets[-1]].copy_(pinned[begin:offsets[-1]], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[turn] = event

    # ------------------------------------------------------------------ graphs
    def length_bounds(self, packed: PackedStep) -> tuple[int, int]:
        """The bound on sequence lengths that the step's launches are sized for, and the middle of the lengths
        that share this bound (0 where the bound is not one of a decode step)."""
        longest = self.cache.max_seq_len
        if not packed.all_single:
            return longest, 0
        below, bound = 0, self.MIN_LENGTH_BOUND
        while bound < packed.max_kv_len:
            # 1, 1.5, 2, 3, 4, 6, ... times the least bound
            below, bound = bound, (bound * 3 // 2 if bound & (bound - 1) == 0 else bound * 4 // 3)
        bound = min(bound, longest)
        return bound, max(1, (below + bound + 1) // 2)

    def length_bound(self, packed: PackedStep) -> int:
        return self.length_bounds(packed)[0]

    def key_of(self, packed: PackedStep) -> tuple:
        if packed.all_single:
            return (packed.n_tokens, packed.n_seqs, packed.n_want, 1, self.length_bound(packed))
        return (packed.n_tokens, packed.n_seqs, packed.n_want, packed.max_q_len, 0)

    def wants_graph(self, packed: PackedStep) -> bool:
        """Decode shapes always; other shapes from their second appearance on."""
        key = self.key_of(packed)
        if key in self.graphs or packed.all_single:
            return True
        if key in self.seen:
            return True
        self.seen.add(key)
        if len(self.seen) > 4096:
            self.seen.clear()
        return False

    def run(self, packed: PackedStep, device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Logits ``[n_want, vocab]``.  The returned tensor is the graph's own output buffer: the next
        replay of the same shape overwrites it."""
        key = self.key_of(packed)
        self.upload(packed, skip_tokens=device_tokens is not None)
        if device_tokens is not None:
            self.meta[0:packed.n_tokens].copy_(device_tokens)
        if key not in self.graphs:
            return self._capture(key, packed)
        self.graphs.move_to_end(key)
        graph, logits = self.graphs[key]
        graph.replay()
        from ..ops import library

        library.launch_count += self.launches[key]
        return logits

    def _capture(self, key: tuple, packed: PackedStep) -> torch.Tensor:
        """Runs the step launch by launch, captures its launches for the steps to come, and returns the
        logits of the run (the capture itself executes nothing, so the step has run once)."""
        from ..ops import library

        self.model.prepare(self.cache.max_seq_len - 1)
        # launch shapes inside a graph must not depend on the lengths of the day: a bound stands in
        bound, typical = self.length_bounds(packed)
        ctx = context_from_views(packed, self.views(packed), self.model.dtype, max_kv_len=bound, typical_kv_len=typical)
        result = self.model.step(ctx, self.cache)  # one-time set-up happens here, outside the capture
        torch.cuda.synchronize()
        while len(self.graphs) >= self.MAX_PREFILL_GRAPHS + 3 * self.s_max:
            self.graphs.popitem(last=False)
        graph = torch.cuda.CUDAGraph()
        before = set_pdl(self.use_pdl)
        count = library.launch_count
        try:
            with torch.cuda.graph(graph, pool=self.pool):
                logits = self.model.step(ctx, self.cache)
        finally:
            set_pdl(before)
        self.launches[key] = library.launch_count - count
        library.launch_count = count
        if self.pool is None:
            self.pool = graph.pool()
        self.graphs[key] = (graph, logits)
        return result

"""Decode steps replayed from CUDA graphs.

A decode step launches some hundred small kernels; issued one by one from Python they cost
far more host time than device time.  The whole step — embedding to logits — is therefore
captured once per batch size and replayed.  Everything that changes from step to step lives in
device memory that the kernels read (token ids, positions, slots, lengths, the page table), so
one graph serves any set of sequences of that size, at any lengths, in any slots; the host's
work per step is one small pinned copy of those numbers.
"""

from __future__ import annotations

import torch

from ..parts.base import StepContext


class DecodeGraphs:
    RING = 8

    def __init__(self, model, cache, use_pdl: bool = True):
        self.model, self.cache, self.use_pdl = model, cache, use_pdl
        self.n_max = cache.max_seqs
        device = model.device
        n = self.n_max
        # device-side step inputs at fixed addresses: tokens | positions | slots | lengths
        self.meta = torch.zeros(4 * n, dtype=torch.int32, device=device)
        self.arange = torch.arange(n + 1, dtype=torch.int32, device=device)
        self.host = [torch.zeros(4 * n, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.host_np = [h.numpy() for h in self.host]
        self.events = [None] * self.RING
        self.turn = 0
        self.graphs: dict[int, tuple[torch.cuda.CUDAGraph, torch.Tensor]] = {}
        self.pool = None

    def context(self, n: int, max_kv_len: int) -> StepContext:
        big = self.n_max
        ctx = StepContext(
            n_tokens=n, n_seqs=n, dtype=self.model.dtype, tokens=self.meta[0:n], tok_pos=self.meta[big:big + n],
            tok_seq=self.arange[:n], cu_q=self.arange[:n + 1], slots=self.meta[2 * big:2 * big + n],
            kv_len=self.meta[3 * big:3 * big + n], want_rows=self.arange[:n], max_q_len=1, max_kv_len=max_kv_len,
            max_position=max_kv_len - 1, all_single=True,
        )
        # launch shapes inside a graph must not depend on the lengths of the day
        from ..ops.functional import decode_splits

        layout = self.cache.layout.requests
        n_kv = max((r.n_kv_heads for r in layout if hasattr(r, "n_kv_heads")), default=1)
        ctx.extras["decode_splits"] = decode_splits(n, n_kv, self.cache.max_seq_len, self.cache.page_size)
        return ctx

    def upload(self, slots: list[int], past: list[int], tokens: list[int] | None) -> None:
        """Puts the step's numbers where the captured kernels read them (one pinned copy)."""
        n, big = len(slots), self.n_max
        turn = self.turn
        self.turn = (turn + 1) % self.RING
        if self.events[turn] is not None:
            self.events[turn].synchronize()  # the copy that last used this buffer has been done
        buf = self.host_np[turn]
        if tokens is not None:
            buf[0:n] = tokens
        buf[big:big + n] = past
        buf[2 * big:2 * big + n] = slots
        buf[3 * big:3 * big + n] = [p + 1 for p in past]
        if tokens is not None:
            self.meta.copy_(self.host[turn], non_blocking=True)
        else:
            self.meta[big:].copy_(self.host[turn][big:], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[turn] = event

    def run(self, slots: list[int], past: list[int], tokens: list[int] | None,
            device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Logits ``[n, vocab]`` of one token per sequence.  The returned tensor is the graph's own
        output buffer: the next replay of the same batch size overwrites it."""
        n = len(slots)
        self.upload(slots, past, tokens)
        if device_tokens is not None:
            self.meta[0:n].copy_(device_tokens)
        if n not in self.graphs:
            self.model.prepare(self.cache.max_seq_len - 1)
            ctx = self.context(n, self.cache.max_seq_len)
            self.model.step(ctx, self.cache)  # a plain run first: one-time set-up must not be captured
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            # Inside the graph every kernel is launched with programmatic stream serialization: it may
            # start (and fetch weights) while the kernel before it drains, and waits for that kernel's
            # results only where it first needs them.
            from ..ops.functional import set_pdl

            before = set_pdl(self.use_pdl)
            try:
                with torch.cuda.graph(graph, pool=self.pool):
                    logits = self.model.step(ctx, self.cache)
            finally:
                set_pdl(before)
            if self.pool is None:
                self.pool = graph.pool()
            self.graphs[n] = (graph, logits)
        graph, logits = self.graphs[n]
        graph.replay()
        return logits

"""The engine: a model, its cache, and the one step function that everything above uses
(generation, trace replay, the benchmark).

It is the successor of the reference's ``Engine`` + model call (src/engine.py:15-46,
src/models/transformer.py:99-101), with three differences that the reference's design cannot
express: sequences of a batch have their own lengths, logits are computed only at the wanted
places, and a sequence that ends gives its storage back while the others go on.
"""

from __future__ import annotations

import array
import os
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import Cache, CacheFull
from ..models.model import Model
from .step import SequenceStep, pack_step, plan_step


def _token_array(tokens) -> np.ndarray:
    """The ids as an int64 array.  A list of Python ints goes through ``array.array`` (about half the time of
    ``np.asarray`` for a prompt of a few thousand tokens); anything else, or a list that holds other things, takes
    numpy's own conversion and its errors."""
    if type(tokens) is list:
        try:
            return np.frombuffer(array.array("q", tokens), dtype=np.int64)
        except (TypeError, OverflowError):
            pass
    return np.asarray(tokens, dtype=np.int64)


@dataclass
class StepEntry:
    """A request's part of a step: its next tokens and the places among them whose logits are wanted."""

    id: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)


class Engine:
    def __init__(self, model: Model, max_tokens: int, max_seqs: int | None = None, use_graphs: bool = True,
                 use_pdl: bool | None = None):
        self.model = model
        self.cache: Cache = model.make_cache(max_tokens, max_seqs)
        self.slot_of: dict[object, int] = {}
        self.steps_run = 0
        self.graphs = None
        if use_graphs and model.device.type == "cuda" and model.graph_safe():
            from .graphs import StepGraphs

            if use_pdl is None:
                use_pdl = os.environ.get("GTAR_B200_PDL", "1") != "0"
            self.graphs = StepGraphs(model, self.cache, use_pdl)

    # ------------------------------------------------------------------ requests
    def live(self) -> list[object]:
        return list(self.slot_of)

    def length(self, request_id) -> int:
        return self.cache.length[self.slot_of[request_id]]

    def end(self, request_ids) -> None:
        """The listed requests are finished: their slots and pages are given back."""
        for request_id in request_ids:
            if request_id not in self.slot_of:
                raise KeyError(f"request {request_id!r} is not live")
            self.cache.close(self.slot_of.pop(request_id))

    def end_all(self) -> None:
        self.end(list(self.slot_of))

    def check(self) -> None:
        """Raises if a kernel of an earlier step gave up one of its bounded waits (its output is then
        not valid).  Synchronises the device; callers use it where they wait for results anyway."""
        if self.model.device.type == "cuda":
            from ..ops.functional import check_kernel_errors

            check_kernel_errors(self.model.device)

    # ------------------------------------------------------------------ the step
    def step(self, entries: list[StepEntry], keep_output: bool = True) -> torch.Tensor:
        """Runs the entries' tokens as one batch from the cache and returns float32 logits
        ``[n_wanted, vocab]`` in the order of the entries and of each entry's ``want``.

        ``keep_output=False`` allows the result to be a buffer that the next step overwrites (the
        generation loop, which consumes the logits at once, asks for that).

        A request seen for the first time gets a slot; the others continue where they are.
        Nothing is changed when the step cannot run (no slot, not enough pages, a bad token).
        """
        if not entries:
            raise ValueError("a step needs at least one entry")
        ids = [e.id for e in entries]
        if len(set(ids)) != len(ids):
            raise ValueError("a request appears twice in one step")
        vocab = self.model.vocab_size
        # all tokens of the step as one array: checked once, and packed from it
        q_lens = [len(e.tokens) for e in entries]
        if min(q_lens) == 0:
            raise ValueError(f"request {entries[q_lens.index(0)].id!r} brings no token")
        parts = [_token_array(e.tokens) for e in entries]
        if any(part.ndim != 1 for part in parts):
            raise ValueError("tokens must be a flat list of ids")
        flat = parts[0] if len(parts) == 1 else np.concatenate(parts)
        if flat.min() < 0 or flat.max() >= vocab:
            for entry, part in zip(entries, parts):
                wrong = part[(part < 0) | (part >= vocab)]
                if wrong.size:
                    raise ValueError(f"request {entry.id!r}: token id {int(wrong[0])} is outside the vocabulary of {vocab}")
        for entry, n in zip(entries, q_lens):
            for place in entry.want:
                if not 0 <= int(place) < n:
                    raise ValueError(f"request {entry.id!r}: wanted place {place} is outside the {n} tokens it brings")
        new_ids = [e.id for e in entries if e.id not in self.slot_of]
        if len(new_ids) > self.cache.slots.n_free:
            raise CacheFull(f"{len(new_ids)} new requests but only {self.cache.slots.n_free} free slots")
        opened = []
        try:
            for request_id in new_ids:
                slot = self.cache.open()
                self.slot_of[request_id] = slot
                opened.append(request_id)
            growth = {self.slot_of[e.id]: len(e.tokens) for e in entries}
            if not self.cache.can_grow(growth):
                raise CacheFull(
                    f"the step's {sum(growth.values())} tokens do not fit: the cache holds "
                    f"{self.cache.n_pages * self.cache.page_size} tokens in pages of {self.cache.page_size} and "
                    f"sequences up to {self.cache.max_seq_len}")
        except Exception:
            for request_id in opened:
                self.cache.close(self.slot_of.pop(request_id))
            raise
        sequences = []
        for entry, tokens in zip(entries, parts):
            slot = self.slot_of[entry.id]
            past = self.cache.grow(slot, len(tokens))
            sequences.append(SequenceStep(slot, past, tokens, [int(w) for w in entry.want]))
        self.cache.sync()
        self.steps_run += 1
        if self.graphs is not None:
            packed = pack_step(sequences, vocab, check_tokens=False)
            if packed.n_want > 0 and self.graphs.wants_graph(packed):
                logits = self.graphs.run(packed)
                return logits.clone() if keep_output else logits
        ctx = plan_step(sequences, self.model.dtype, self.model.device, vocab)
        return self.model.step(ctx, self.cache)

    def decode_on_device(self, request_ids: list, tokens: torch.Tensor) -> torch.Tensor:
        """One token for each of the listed live requests, the token ids being on the device already
        (int32 ``[n]``, for instance the sampler's output): no token crosses to the host.  Returns
        float32 logits ``[n, vocab]`` in a buffer that the next step may overwrite.  The ids are
        trusted to lie inside the vocabulary."""
        if tokens.dtype != torch.int32 or tokens.dim() != 1 or tokens.shape[0] != len(request_ids):
            raise ValueError("tokens must be int32 [n] with one entry per request")
        slots = [self.slot_of[r] for r in request_ids]
        growth = {slot: 1 for slot in slots}
        if len(growth) != len(slots):
            raise ValueError("a request appears twice in one step")
        if not self.cache.can_grow(growth):
            raise CacheFull("no room in the cache for one more token of every request")
        sequences = [SequenceStep(slot, self.cache.grow(slot, 1), [0], [0]) for slot in slots]
        self.cache.sync()
        self.steps_run += 1
        if self.graphs is not None:
            return self.graphs.run(pack_step(sequences, self.model.vocab_size, check_tokens=False), device_tokens=tokens)
        ctx = plan_step(sequences, self.model.dtype, self.model.device, self.model.vocab_size, device_tokens=tokens)
        return self.model.step(ctx, self.cache)

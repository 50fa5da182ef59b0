"""The generation loop: batches of unequal prompts, one token per live sequence per step, stop
tokens, sequences that end earlier, one batch after another until every request is served.

The reference's loop (src/engine.py:30-46) takes one rectangular batch, keeps finished rows in
it (feeding them EOS) until all are finished, and never feeds the last sampled token back.  This
loop keeps the last rule and the emitted-stop-token rule (the stop token is part of the output,
src/engine.py:39-42) and differs where the reference cannot: prompts may differ in length, a
finished sequence leaves the batch at once and frees its storage, and requests beyond one
batch's room wait for the next batch.

The loop's decisions are plain host code over two callables — ``engine.step`` /
``engine.end`` and a chooser that turns logits into token ids — so they can be tested with
stand-ins for both.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Sequence

from .engine import StepEntry


@dataclass(frozen=True)
class GenerationParams:
    max_new_tokens: int = 64  # the reference's command-line default (scripts/generate.py:24)
    stop_ids: frozenset = frozenset()
    max_batch: int = 64  # most sequences decoded together

    def __post_init__(self):
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")
        if self.max_batch <= 0:
            raise ValueError("max_batch must be positive")


@dataclass
class _Live:
    index: int  # position of the request in the call
    request_id: object
    produced: list[int] = field(default_factory=list)


def round_up(n: int, unit: int) -> int:
    return -(-n // unit) * unit


def form_batches(prompt_lens: Sequence[int], max_new_tokens: int, max_batch: int, token_room: int, unit: int,
                 max_seq_len: int | None, slot_room: int) -> list[list[int]]:
    """Splits request indices ``0..n-1`` into consecutive batches.  A request reserves
    ``prompt + max_new_tokens - 1`` positions (the last chosen token is never fed back) rounded
    up to the cache's page ``unit``; a batch takes requests in order while they fit in
    ``token_room`` tokens, ``slot_room`` slots and ``max_batch`` sequences."""
    batches: list[list[int]] = []
    current: list[int] = []
    used = 0
    for index, n_prompt in enumerate(prompt_lens):
        if n_prompt <= 0:
            raise ValueError(f"request {index} has an empty prompt")
        need = n_prompt + max(0, max_new_tokens - 1)
        if max_seq_len is not None:
            if n_prompt > max_seq_len:
                raise ValueError(f"request {index}: prompt of {n_prompt} tokens exceeds the longest sequence ({max_seq_len})")
            need = min(need, max_seq_len)
        need = round_up(need, unit)
        if need > token_room:
            raise ValueError(f"request {index} needs room for {need} tokens; the cache holds {token_room}")
        if current and (len(current) >= min(max_batch, slot_room) or used + need > token_room):
            batches.append(current)
            current, used = [], 0
        current.append(index)
        used += need
    if current:
        batches.append(current)
    return batches


Chooser = Callable[[object, list[int], list[int]], list[int]]  # (logits, request indices, steps) -> token ids


def run_generation(engine, prompts: Sequence[Sequence[int]], params: GenerationParams, choose: Chooser,
                   request_offset: int = 0, on_step: Callable | None = None) -> list[list[int]]:
    """Generates for every prompt; returns the new tokens of each (the stop token included).

    ``engine`` offers ``step(entries) -> logits`` and ``end(ids)``, and a ``cache`` with
    ``n_pages``, ``page_size``, ``max_seq_len`` and ``max_seqs``.
    """
    outputs: list[list[int]] = [[] for _ in prompts]
    if params.max_new_tokens == 0 or not prompts:
        return outputs
    cache = engine.cache
    batches = form_batches([len(p) for p in prompts], params.max_new_tokens, params.max_batch,
                           cache.n_pages * cache.page_size, cache.page_size, cache.max_seq_len, cache.max_seqs)
    for batch in batches:
        live = [_Live(i, ("gen", request_offset + i)) for i in batch]
        entries = [StepEntry(s.request_id, list(prompts[s.index]), [len(prompts[s.index]) - 1]) for s in live]
        try:
            while live:
                logits = engine.step(entries, keep_output=False)
                tokens = choose(logits, [request_offset + s.index for s in live], [len(s.produced) for s in live])
                if on_step is not None:
                    on_step(live, tokens)
                still: list[_Live] = []
                ended: list[object] = []
                for seq, token in zip(live, tokens):
                    token = int(token)
                    seq.produced.append(token)
                    length_after = len(prompts[seq.index]) + len(seq.produced)  # if the token were fed back
                    done = (
                        token in params.stop_ids
                        or len(seq.produced) >= params.max_new_tokens
                        or (cache.max_seq_len is not None and length_after > cache.max_seq_len)
                    )
                    if done:
                        ended.append(seq.request_id)
                        outputs[seq.index] = seq.produced
                    else:
                        still.append(seq)
                if ended:
                    engine.end(ended)
                live = still
                entries = [StepEntry(s.request_id, [s.produced[-1]], [0]) for s in live]
        except Exception:
            leftover = [s.request_id for s in live if s.request_id in getattr(engine, "slot_of", {})]
            if leftover:
                engine.end(leftover)
            raise
    return outputs

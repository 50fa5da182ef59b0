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


@dataclass
class DeviceChooser:
    """The chooser in two halves, for an engine that can take a step's tokens from device memory:
    ``choose(logits, request indices, steps)`` returns the token ids as a device tensor (int32 ``[n]``),
    ``fetch(tokens)`` starts their copy to the host and returns a callable that waits for it and gives the
    list.  With both, the next step is launched on the device's copy of the tokens before the host has
    seen them, and the host's work on a step (stop tokens, bookkeeping, the next step's numbers) happens
    while the device computes."""

    choose: Callable
    fetch: Callable
    take: Callable  # (tokens on the device, row indices) -> those rows, on the device


def run_generation(engine, prompts: Sequence[Sequence[int]], params: GenerationParams, choose: Chooser,
                   request_offset: int = 0, on_step: Callable | None = None,
                   device_chooser: DeviceChooser | None = None) -> list[list[int]]:
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
    if device_chooser is not None and hasattr(engine, "decode_on_device"):
        for batch in batches:
            _run_batch_ahead(engine, prompts, params, device_chooser, request_offset, on_step, batch, outputs)
        return outputs
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


def _run_batch_ahead(engine, prompts, params: GenerationParams, chooser: DeviceChooser, request_offset: int,
                     on_step: Callable | None, batch: list[int], outputs: list[list[int]]) -> None:
    """One batch with the device one step ahead of the host.

    The tokens a step chose stay on the device and are fed to the next step at once, for every sequence
    that may go on (one that has reached ``max_new_tokens`` or the longest sequence certainly does not);
    only then does the host wait for the step's tokens.  A sequence that turns out to have chosen a stop
    token has been fed one step too many: that step's token for it is dropped, and its storage is given
    back like any other's.  The tokens a sequence gets are the same as in the loop above.
    """
    cache = engine.cache
    live = [_Live(i, ("gen", request_offset + i)) for i in batch]
    try:
        entries = [StepEntry(s.request_id, list(prompts[s.index]), [len(prompts[s.index]) - 1]) for s in live]
        logits = engine.step(entries, keep_output=False)
        rows = list(live)  # rows[i]: the sequence row i of the pending step's tokens belongs to
        tokens_dev = chooser.choose(logits, [request_offset + s.index for s in rows], [0] * len(rows))
        wait = chooser.fetch(tokens_dev)
        while rows:
            # --- the next step, on the device's copy of the pending tokens
            def may_go_on(seq: _Live) -> bool:  # after the pending token
                n = len(seq.produced) + 1
                fed_length = len(prompts[seq.index]) + n
                return n < params.max_new_tokens and not (cache.max_seq_len is not None and fed_length > cache.max_seq_len)
            keep = [i for i, seq in enumerate(rows) if may_go_on(seq)]
            next_rows, next_tokens_dev, next_wait = [], None, None
            if keep:
                next_rows = [rows[i] for i in keep]
                fed = tokens_dev if len(keep) == len(rows) else chooser.take(tokens_dev, keep)
                logits = engine.decode_on_device([s.request_id for s in next_rows], fed)
                next_tokens_dev = chooser.choose(logits, [request_offset + s.index for s in next_rows],
                                                 [len(s.produced) + 1 for s in next_rows])
                next_wait = chooser.fetch(next_tokens_dev)
            # --- the pending step's tokens on the host
            tokens = wait()
            if on_step is not None:
                on_step(rows, tokens)
            ended = []
            for seq, token in zip(rows, tokens):
                token = int(token)
                seq.produced.append(token)
                length_after = len(prompts[seq.index]) + len(seq.produced)
                if (token in params.stop_ids or len(seq.produced) >= params.max_new_tokens
                        or (cache.max_seq_len is not None and length_after > cache.max_seq_len)):
                    ended.append(seq)
                    outputs[seq.index] = seq.produced
            if ended:
                engine.end([s.request_id for s in ended])
                live = [s for s in live if s not in ended]
                gone = set(id(s) for s in ended)
                if any(id(s) in gone for s in next_rows):  # fed one step too many: their rows of the next step are dropped
                    still = [i for i, s in enumerate(next_rows) if id(s) not in gone]
                    next_rows = [next_rows[i] for i in still]
                    if next_rows:
                        next_wait = _subset(next_wait, still)
                        next_tokens_dev = chooser.take(next_tokens_dev, still)
            rows, tokens_dev, wait = next_rows, next_tokens_dev, next_wait
    except Exception:
        leftover = [s.request_id for s in live if s.request_id in getattr(engine, "slot_of", {})]
        if leftover:
            engine.end(leftover)
        raise


def _subset(wait: Callable, keep: list[int]) -> Callable:
    def waited():
        tokens = wait()
        return [tokens[i] for i in keep]
    return waited

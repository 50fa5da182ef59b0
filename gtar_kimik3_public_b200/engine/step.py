"""The step function's host side: turns a batch of (sequence, new tokens, wanted places) into
the device tensors the kernels read, with one host-to-device copy.

The reference's model call is rectangular: every row has the same number of cached and new
tokens (src/models/transformer.py:60-63).  A step here carries sequences with their own
``past`` and ``new`` counts; the rule for what a token sees is the reference's, per sequence:
key ``j`` is visible to new token ``i`` iff ``j <= past + i`` (src/layers/attention.py:116-119).
"""

from __future__ import annotations

from dataclasses import dataclass

from typing import Sequence

import numpy as np
import torch

from ..parts.base import StepContext


@dataclass
class SequenceStep:
    """One sequence's part of a step."""

    slot: int
    past_len: int
    tokens: Sequence[int]  # a list or a numpy array of ids
    want: list[int]  # places among ``tokens`` whose logits are asked for


@dataclass
class PackedStep:
    """The numbers of a step on the host, in the order they are laid out for the device:
    tokens | positions | sequence of each token | starts | slots | lengths | wanted rows."""

    fields: list[np.ndarray]
    q_lens: list[int]
    past: list[int]
    slots: list[int]

    @property
    def n_tokens(self) -> int:
        return len(self.fields[0])

    @property
    def n_seqs(self) -> int:
        return len(self.slots)

    @property
    def n_want(self) -> int:
        return len(self.fields[6])

    @property
    def all_single(self) -> bool:
        return self.n_tokens == self.n_seqs

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens)

    @property
    def max_kv_len(self) -> int:
        return max(p + n for p, n in zip(self.past, self.q_lens))


def pack_step(sequences: list[SequenceStep], vocab_size: int, check_tokens: bool = True) -> PackedStep:
    if not sequences:
        raise ValueError("a step needs at least one sequence")
    q_lens = [len(s.tokens) for s in sequences]
    if min(q_lens) == 0:
        raise ValueError(f"sequence {q_lens.index(0)} of the step brings no token")
    past = [s.past_len for s in sequences]
    n_seqs = len(sequences)
    past_np = np.asarray(past, dtype=np.int32)
    if n_seqs == 1 and q_lens[0] > 1:  # one prompt (or continuation): nothing to repeat or add up
        n = q_lens[0]
        starts = np.array([0, n], dtype=np.int32)
        tokens = np.asarray(sequences[0].tokens, dtype=np.int64)
        tok_seq = np.zeros(n, dtype=np.int32)
        tok_pos = np.arange(past[0], past[0] + n, dtype=np.int32)
    elif max(q_lens) == 1:  # a decode step: one token each
        starts = np.arange(n_seqs + 1, dtype=np.int32)
        tokens = np.asarray([s.tokens[0] for s in sequences], dtype=np.int64)
        tok_seq, tok_pos = starts[:-1], past_np
    else:
        starts = np.zeros(n_seqs + 1, dtype=np.int32)
        np.cumsum(q_lens, out=starts[1:])
        tokens = np.concatenate([np.asarray(s.tokens, dtype=np.int64) for s in sequences])
        tok_seq = np.repeat(np.arange(n_seqs, dtype=np.int32), q_lens)
        tok_pos = np.arange(int(starts[-1]), dtype=np.int32) - starts[:-1][tok_seq] + past_np[tok_seq]
    if check_tokens and tokens.size and (tokens.min() < 0 or tokens.max() >= vocab_size):
        bad = int(tokens[(tokens < 0) | (tokens >= vocab_size)][0])
        raise ValueError(f"token id {bad} is outside the vocabulary of {vocab_size}")
    want_rows = []
    for index, seq in enumerate(sequences):
        for place in seq.want:
            if not 0 <= place < q_lens[index]:
                raise ValueError(f"wanted place {place} is outside the {q_lens[index]} tokens sequence {index} brings")
            want_rows.append(int(starts[index]) + place)
    slots = [s.slot for s in sequences]
    fields = [
        tokens.astype(np.int32), tok_pos.astype(np.int32), tok_seq, starts, np.asarray(slots, dtype=np.int32),
        past_np + np.asarray(q_lens, dtype=np.int32), np.asarray(want_rows, dtype=np.int32),
    ]
    return PackedStep(fields, q_lens, past, slots)


def context_from_views(packed: PackedStep, views: list[torch.Tensor], dtype: torch.dtype, max_kv_len: int | None = None,
                       device_tokens: torch.Tensor | None = None, typical_kv_len: int = 0) -> StepContext:
    max_kv = packed.max_kv_len if max_kv_len is None else max_kv_len
    return StepContext(
        n_tokens=packed.n_tokens, n_seqs=packed.n_seqs, dtype=dtype,
        tokens=views[0] if device_tokens is None else device_tokens, tok_pos=views[1], tok_seq=views[2], cu_q=views[3],
        slots=views[4], kv_len=views[5], want_rows=views[6], max_q_len=packed.max_q_len, max_kv_len=max_kv,
        max_position=max_kv - 1, all_single=packed.all_single, typical_kv_len=typical_kv_len, host_q_len=packed.q_lens, host_past_len=packed.past,
        host_slots=packed.slots,
    )


def plan_step(sequences: list[SequenceStep], dtype: torch.dtype, device: torch.device, vocab_size: int,
              device_tokens: torch.Tensor | None = None) -> StepContext:
    """Builds the step's context in fresh device memory (one pinned copy).  With ``device_tokens``
    (int32, one per packed token, already on the device — e.g. the sampler's output) the
    sequences' ``tokens`` only give the counts."""
    packed = pack_step(sequences, vocab_size, check_tokens=device_tokens is None)
    flat = torch.from_numpy(np.concatenate(packed.fields))
    if device.type == "cuda":
        flat = flat.pin_memory()
    dev = flat.to(device, non_blocking=True)
    views, start = [], 0
    for f in packed.fields:
        views.append(dev[start:start + len(f)])
        start += len(f)
    return context_from_views(packed, views, dtype, device_tokens=device_tokens)

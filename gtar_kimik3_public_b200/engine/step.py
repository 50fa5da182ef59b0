"""The step function's host side: turns a batch of (sequence, new tokens, wanted places) into
the device tensors the kernels read, with one host-to-device copy.

The reference's model call is rectangular: every row has the same number of cached and new
tokens (src/models/transformer.py:60-63).  A step here carries sequences with their own
``past`` and ``new`` counts; the rule for what a token sees is the reference's, per sequence:
key ``j`` is visible to new token ``i`` iff ``j <= past + i`` (src/layers/attention.py:116-119).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import StepContext


@dataclass
class SequenceStep:
    """One sequence's part of a step."""

    slot: int
    past_len: int
    tokens: list[int]
    want: list[int]  # places among ``tokens`` whose logits are asked for


def plan_step(sequences: list[SequenceStep], dtype: torch.dtype, device: torch.device, vocab_size: int,
              device_tokens: torch.Tensor | None = None) -> StepContext:
    """Builds the step's context.  With ``device_tokens`` (int32, one per packed token, already on
    the device — e.g. the sampler's output) the sequences' ``tokens`` only give the counts."""
    if not sequences:
        raise ValueError("a step needs at least one sequence")
    tokens: list[int] = []
    tok_pos: list[int] = []
    tok_seq: list[int] = []
    cu_q = [0]
    want_rows: list[int] = []
    for index, seq in enumerate(sequences):
        n = len(seq.tokens)
        if n == 0:
            raise ValueError(f"sequence {index} of the step brings no token")
        for place in seq.want:
            if not 0 <= place < n:
                raise ValueError(f"wanted place {place} is outside the {n} tokens sequence {index} brings")
            want_rows.append(cu_q[-1] + place)
        if device_tokens is None:
            for token in seq.tokens:
                if not 0 <= token < vocab_size:
                    raise ValueError(f"token id {token} is outside the vocabulary of {vocab_size}")
        tokens.extend(seq.tokens)
        tok_pos.extend(range(seq.past_len, seq.past_len + n))
        tok_seq.extend([index] * n)
        cu_q.append(cu_q[-1] + n)
    slots = [s.slot for s in sequences]
    kv_len = [s.past_len + len(s.tokens) for s in sequences]
    fields = [tokens, tok_pos, tok_seq, cu_q, slots, kv_len, want_rows]
    flat = torch.tensor([x for f in fields for x in f], dtype=torch.int32)
    if device.type == "cuda":
        flat = flat.pin_memory()
    dev = flat.to(device, non_blocking=True)
    views = []
    start = 0
    for f in fields:
        views.append(dev[start:start + len(f)])
        start += len(f)
    q_lens = [len(s.tokens) for s in sequences]
    return StepContext(
        n_tokens=len(tokens), n_seqs=len(sequences), dtype=dtype,
        tokens=views[0] if device_tokens is None else device_tokens, tok_pos=views[1], tok_seq=views[2], cu_q=views[3], slots=views[4], kv_len=views[5],
        want_rows=views[6], max_q_len=max(q_lens), max_kv_len=max(kv_len), max_position=max(kv_len) - 1,
        all_single=all(n == 1 for n in q_lens), host_q_len=q_lens, host_past_len=[s.past_len for s in sequences], host_slots=slots,
    )

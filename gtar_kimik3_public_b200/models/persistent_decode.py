"""Decode steps of up to eight sequences through ONE persistent kernel for all layers (an option, off by default).

A model qualifies when every entry of its run list is a layer of the one shape the kernel knows: a pre-norm block of
RMSNorm, grouped-query attention (optional per-head q/k norm, optional rotation, all positions kept, storage of its
own), RMSNorm and a SwiGLU feed-forward, with bfloat16 matrices and the same sizes in every layer.  The parts say so
themselves (``decode_record()``); a model with any other part steps through its parts one by one as before.  Nothing
here knows an architecture: the plan is made from the run list and the cache's views.

Measured on a B200 (28 layers of the Qwen3-0.6B sizes, 2,048-token contexts) the persistent kernel takes 1.64 ms a step
for one sequence and 1.81 ms for eight, where the chain of seven kernels a layer takes 0.78 and 1.01 ms: a barrier over
the whole grid costs 1.5 us after the last block has arrived, a stage after it another 3 to 5 us (one trip to L2 for
the activations, the tiles' arithmetic at one warp per scheduler pair, the partial sums, the stores), so that a
layer's five stages cost more than the seven kernel boundaries they replace.  It stays in the tree as an option
(``GTAR_B200_PERSISTENT_DECODE=1`` or ``ENABLED = True``), tested, with clock stamps at every barrier for whoever
takes it further.
"""

from __future__ import annotations

import os
import struct

import torch

from ..ops import functional as F

ENABLED = os.environ.get("GTAR_B200_PERSISTENT_DECODE", "0") == "1"
RECORD_BYTES = 96  # the kernel's record of a layer: ten pointers, three floats, one int


class PersistentDecode:
    """The layer table and the work areas of one (model, cache) pair."""

    def __init__(self, layer_table, n_layers, sizes, work, rope, norm_bf16, qk_bf16, scale):
        self.layer_table, self.n_layers, self.sizes, self.work = layer_table, n_layers, sizes, work
        self.rope, self.norm_bf16, self.qk_bf16, self.scale = rope, norm_bf16, qk_bf16, scale
        self.stamps = None  # a tensor here makes the kernel record when each block reaches and leaves each barrier

    def run(self, h: torch.Tensor, ctx) -> None:
        hidden, n_q, n_kv, head_dim, inter = self.sizes
        cos = sin = None
        if self.rope is not None:
            cos, sin = self.rope.cos, self.rope.sin
        qkv, att, act, part, words, table = self.work
        F.decode_layers(self.layer_table, self.n_layers, h, n_q, n_kv, head_dim, inter, qkv, att, act, part, words,
                        ctx.kv_len, ctx.slots, table, ctx.max_kv_len, cos, sin, self.norm_bf16, self.qk_bf16, self.scale,
                        self.stamps)


def build(model, cache) -> PersistentDecode | None:
    """The plan for this model on this cache, or None if a layer, a size or the cache is not what the kernel takes."""
    if not ENABLED or model.dtype != torch.bfloat16 or model.device.type != "cuda":
        return None
    plan = model.plan
    records, views = [], []
    for index, entry in enumerate(plan.run_list):
        describe = getattr(plan.layers[entry.layer], "decode_record", None)
        record = describe() if describe is not None else None
        view = cache.view(index)
        if record is None or cache.is_shared(index) or not isinstance(view, F.PagedKV):
            return None
        records.append(record)
        views.append(view)
    first = records[0]
    same = ("hidden", "n_q", "n_kv", "head_dim", "inter", "rope", "norm_dtype", "qk_dtype", "scale", "has_qk_norm")
    if any(r[key] is not first[key] and r[key] != first[key] for r in records for key in same):
        return None
    if any(view.block_table.data_ptr() != views[0].block_table.data_ptr() or view.k.dtype != torch.bfloat16 for view in views):
        return None  # layers of different cache groups have page tables of their own
    sizes = (first["hidden"], first["n_q"], first["n_kv"], first["head_dim"], first["inter"])
    need = F.decode_layers_work_sizes(F.DECODE_LAYERS_MAX_SEQS, *sizes, cache.max_seq_len, cache.page_size)
    if need is None:
        return None
    device = model.device
    packed = bytearray()
    for record, view in zip(records, views):
        pointers = [record["w_qkv"], record["w_o"], record["w_gu"], record["w_down"], record["norm_in"], record["norm_post"],
                    record["q_norm"], record["k_norm"]]
        packed += struct.pack("<10Q3fi", *[0 if t is None else t.data_ptr() for t in pointers], view.k.data_ptr(),
                              view.v.data_ptr(), record["eps_in"], record["eps_post"], record["eps_qk"], 0)
    assert len(packed) == RECORD_BYTES * len(records)
    layer_table = torch.frombuffer(packed, dtype=torch.uint8).to(device)
    n_seqs = F.DECODE_LAYERS_MAX_SEQS
    hidden, n_q, n_kv, head_dim, inter = sizes
    work = (
        torch.empty(n_seqs * (n_q + 2 * n_kv) * head_dim, dtype=torch.bfloat16, device=device),
        torch.empty(n_seqs * n_q * head_dim, dtype=torch.bfloat16, device=device),
        torch.empty(n_seqs * inter, dtype=torch.bfloat16, device=device),
        torch.empty(need[0], dtype=torch.float32, device=device),
        torch.zeros(need[1], dtype=torch.int32, device=device),
        views[0].block_table,
    )
    return PersistentDecode(layer_table, len(records), sizes, work, first["rope"], first["norm_dtype"] == torch.bfloat16,
                            first["qk_dtype"] == torch.bfloat16, first["scale"])

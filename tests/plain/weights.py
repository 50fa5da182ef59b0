"""Seeded random weights and a safetensors reader of the tests' own.

``make_weights`` follows the layout of the reference's state dict (probe of
``TransformerForCausalLM(...).state_dict().keys()``, src/models/transformer.py:52-77): the
embedding, eleven tensors per layer, the final norm and the head.  Values: matrices
N(0, std), norm weights 1 + N(0, 0.1) so that a forgotten norm weight shows.
``read_safetensors`` parses the file format by hand so that the tests do not lean on the
library's reader.
"""

from __future__ import annotations

import json
import struct

import numpy as np
import torch


def tensor_names(cfg: dict) -> list[tuple[str, tuple[int, ...], str]]:
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    names = [("model.embed_tokens.weight", (v, h), "matrix")]
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        names += [
            (p + "self_attn.q_proj.weight", (nq * d, h), "matrix"),
            (p + "self_attn.k_proj.weight", (nkv * d, h), "matrix"),
            (p + "self_attn.v_proj.weight", (nkv * d, h), "matrix"),
            (p + "self_attn.o_proj.weight", (h, nq * d), "matrix"),
            (p + "self_attn.q_norm.weight", (d,), "norm"),
            (p + "self_attn.k_norm.weight", (d,), "norm"),
            (p + "mlp.gate_proj.weight", (i, h), "matrix"),
            (p + "mlp.up_proj.weight", (i, h), "matrix"),
            (p + "mlp.down_proj.weight", (h, i), "matrix"),
            (p + "input_layernorm.weight", (h,), "norm"),
            (p + "post_attention_layernorm.weight", (h,), "norm"),
        ]
    names.append(("model.norm.weight", (h,), "norm"))
    if not cfg["tie_word_embeddings"]:
        names.append(("lm_head.weight", (v, h), "matrix"))
    return names


def make_weights(cfg: dict, seed: int, std: float = 0.02, round_to_bf16: bool = True) -> dict[str, torch.Tensor]:
    """float32 tensors; with ``round_to_bf16`` the matrices hold values bfloat16 can store exactly."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape, kind in tensor_names(cfg):
        if kind == "matrix":
            t = torch.randn(shape, generator=gen) * std
            if round_to_bf16:
                t = t.to(torch.bfloat16).to(torch.float32)
        else:
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
        out[name] = t
    return out


_NP = {"F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64, "F16": np.float16}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """All tensors of one file as float32/int tensors (bfloat16 widened exactly)."""
    with open(path, "rb") as handle:
        (n,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(n))
        data = handle.read()
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        raw = data[begin:end]
        if entry["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = bits.view(np.float32)
        else:
            arr = np.frombuffer(raw, dtype=_NP[entry["dtype"]])
        out[name] = torch.from_numpy(arr.copy()).reshape(entry["shape"])
    return out

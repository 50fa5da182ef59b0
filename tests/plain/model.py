"""A plain, slow implementation of the Qwen3-style dense decoder, written from the reference's
formulas.  Whole sequences, no cache, one function for each part, PyTorch on the CPU (or, for the
tests at real layer sizes, the same lines on the device that holds the tensors it is given).

It shares no code with the library under test: it reads a dict of tensors keyed by the
reference's state-dict names and a dict of config values, nothing else.  Every function
cites the reference lines (paths inside qtris123/gtar-kimik3-public) that it restates.

Agreement of this file with the reference's own model code was checked once on tiny random
models; the outputs of that run are under ``tests/golden/`` with the script that made them
(``tests/golden/make_golden.py``) and ``tests/test_plain_golden.py`` checks them on every run.
"""

from __future__ import annotations

import torch

# When set to torch.bfloat16, every matrix product rounds its operands and its result to that
# type while norms, rotation, softmax and the residual stream stay in the working precision:
# what the reference does on a GPU under torch.autocast (src/engine.py:35).  It is the "standard
# low-precision implementation" whose error the bfloat16 tests measure the library against.
LOWP: torch.dtype | None = None


def mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a @ b, optionally with operands and result rounded to LOWP."""
    if LOWP is None:
        return a @ b
    wide = a.dtype
    return (a.to(LOWP).to(wide) @ b.to(LOWP).to(wide)).to(LOWP).to(wide)


def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h0[t] = E[ids[t]]  — src/models/transformer.py:55,61 (no scale, no position added)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """weight * (x * rsqrt(mean(x^2, -1) + eps))  — src/layers/rmsnorm.py:11-16.

    eps sits inside the square root and is added to the mean; the weight multiplies last.
    """
    variance = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rotary_tables(positions: torch.Tensor, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin of  pos * inv_freq,  inv_freq[i] = 1 / theta^(2i/d)  — src/layers/rope.py:8,11-14.

    inv_freq is built in float32 by the reference's expression; the angle is a float32 product.
    Returned tables are [T, d] with the d/2 angles repeated twice (cat(freqs, freqs)).
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = positions.to(torch.float32)[:, None] * inv_freq.to(positions.device)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """cat(-x[d/2:], x[:d/2])  — src/layers/rope.py:17-19 (pairs (i, i + d/2), not interleaved)."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin  — src/layers/rope.py:29-33.  x: [T, heads, d]; cos, sin: [T, d]."""
    cos = cos[:, None, :].to(x.dtype)
    sin = sin[:, None, :].to(x.dtype)
    return x * cos + rotate_half(x) * sin


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """softmax over the visible keys of (q . k) * d^-0.5, times v.

    q: [T, n_q, d]; k, v: [T, n_kv, d] (the whole sequence, so past = 0).  Query head hq reads
    kv head hq // (n_q // n_kv)  — src/ops/flash_attention_2.py:33-34.  Key j is visible to
    query i iff j <= i  — src/layers/attention.py:116-119 with past_len = 0.  Scale is
    head_dim ** -0.5  — src/ops/flash_attention_2.py:216.  ``window`` (not part of the
    reference's architecture; used by kernel tests only) further hides keys j <= i - window.
    """
    n_tokens, n_q, d = q.shape
    n_kv = k.shape[1]
    group = n_q // n_kv
    out = torch.empty_like(q)
    idx = torch.arange(n_tokens, device=q.device)
    visible = idx[None, :] <= idx[:, None]
    if window:
        visible &= idx[None, :] > idx[:, None] - window
    for hq in range(n_q):
        hk = hq // group
        scores = mm(q[:, hq, :], k[:, hk, :].T) * (d**-0.5)
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, hq, :] = mm(torch.softmax(scores, dim=-1), v[:, hk, :])
    return out


def attention_mixer(x: torch.Tensor, w: dict[str, torch.Tensor], prefix: str, cfg: dict) -> torch.Tensor:
    """Projections, per-head q/k RMSNorm, rotary, attention, output projection.

    src/layers/attention.py:79-89,114-121: q/k/v = x W^T viewed as [T, heads, d]; q_norm and
    k_norm are RMSNorms over d with one [d] weight shared by all heads, applied before the
    rotation; v is neither normed nor rotated; heads are merged and multiplied by Wo^T.
    """
    n_q, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    n_tokens = x.shape[0]
    q = mm(x, w[prefix + "q_proj.weight"].T).view(n_tokens, n_q, d)
    k = mm(x, w[prefix + "k_proj.weight"].T).view(n_tokens, n_kv, d)
    v = mm(x, w[prefix + "v_proj.weight"].T).view(n_tokens, n_kv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    cos, sin = rotary_tables(torch.arange(n_tokens, device=x.device), d, cfg["rope_theta"])
    q = apply_rotary(q, cos, sin)
    k = apply_rotary(k, cos, sin)
    o = causal_gqa_attention(q, k, v)
    return mm(o.reshape(n_tokens, n_q * d), w[prefix + "o_proj.weight"].T)


def swiglu(x: torch.Tensor, w: dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)),  silu(z) = z * sigmoid(z)  — src/layers/swiglu.py:9-14."""
    gate = mm(x, w[prefix + "gate_proj.weight"].T)
    up = mm(x, w[prefix + "up_proj.weight"].T)
    return mm((gate * torch.sigmoid(gate)) * up, w[prefix + "down_proj.weight"].T)


def block(h: torch.Tensor, w: dict[str, torch.Tensor], layer: int, cfg: dict) -> torch.Tensor:
    """h += attn(ln_in(h)); h += mlp(ln_post(h))  — src/models/transformer.py:47-48."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = h + attention_mixer(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", cfg)
    h = h + swiglu(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return h


def forward(ids: torch.Tensor, w: dict[str, torch.Tensor], cfg: dict, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Logits [T, V] of one whole sequence: embedding, the blocks in order, the final norm, the
    head  — src/models/transformer.py:60-67,99-101.  A tied head multiplies by the embedding
    table (transformer.py:76-77)."""
    w = {name: tensor.to(dtype) for name, tensor in w.items()}
    ids = ids.to(w["model.embed_tokens.weight"].device)
    h = embed(ids, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        h = block(h, w, layer, cfg)
    z = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return mm(z, head.T)


def greedy_generate(prompt: list[int], w: dict, cfg: dict, max_new_tokens: int, stop_ids=(),
                    dtype: torch.dtype = torch.float32) -> list[int]:
    """Greedy decoding by running the whole sequence again for every token: argmax of the last
    position's logits, appended; a stop token is emitted and ends the sequence
    (src/engine.py:36-45; the lowest index wins a tie, as torch.argmax does)."""
    ids = list(prompt)
    out: list[int] = []
    for _ in range(max_new_tokens):
        logits = forward(torch.tensor(ids), w, cfg, dtype)[-1]
        token = int(torch.argmax(logits))
        out.append(token)
        if token in stop_ids:
            break
        ids.append(token)
    return out

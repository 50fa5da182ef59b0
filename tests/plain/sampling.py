"""Plain token choice: what the library's samplers must reproduce.

The reference (src/engine.py:5-12): temperature 0 means argmax; otherwise logits / temperature,
an optional top-k mask that keeps every value >= the k-th largest (ties at the threshold
survive), softmax, and one multinomial draw.  The draw here uses the Gumbel-max rule, which
samples from the same distribution as multinomial(softmax(.)): argmax_i (logit_i / T + g_i),
g_i = -log(-log(u_i)).  The uniforms come from a counter-based generator keyed by
(seed, request, step, index), written here with numpy's wrapping uint64 arithmetic.
"""

from __future__ import annotations

import numpy as np

_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_GOLD = np.uint64(0x9E3779B97F4A7C15)


def uniforms(seed: int, request: int, step: int, n: int) -> np.ndarray:
    """n float32 uniforms in (0, 1): splitmix64 finaliser of a linear key, top 23 bits + 1/2."""
    with np.errstate(over="ignore"):
        x = (np.uint64(seed) * _GOLD + np.uint64(request) * _M1 + np.uint64(step) * _M2
             + np.arange(n, dtype=np.uint64))
        x ^= x >> np.uint64(30)
        x *= _M1
        x ^= x >> np.uint64(27)
        x *= _M2
        x ^= x >> np.uint64(31)
    return ((x >> np.uint64(41)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def greedy(logits: np.ndarray) -> int:
    """argmax, lowest index on ties  — src/engine.py:6-7."""
    return int(np.argmax(logits))


def top_k_mask(logits: np.ndarray, top_k: int | None) -> np.ndarray:
    """Boolean mask of the values that survive  — src/engine.py:9-11 (logits < cutoff are dropped)."""
    if not top_k or top_k >= logits.shape[-1]:
        return np.ones_like(logits, dtype=bool)
    cutoff = np.sort(logits)[-top_k]
    return logits >= cutoff


def sample(logits: np.ndarray, temperature: float, top_k: int | None, seed: int, request: int, step: int) -> int:
    logits = np.asarray(logits, dtype=np.float32)
    if temperature == 0:
        return greedy(logits)
    keep = top_k_mask(logits, top_k)
    u = uniforms(seed, request, step, logits.shape[-1])
    gumbel = -np.log(-np.log(u))
    scores = logits / np.float32(temperature) + gumbel.astype(np.float32)
    scores = np.where(keep, scores, -np.inf)
    return int(np.argmax(scores))

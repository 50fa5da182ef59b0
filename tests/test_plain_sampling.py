"""The plain sampler itself: the rule it states (argmax of logits/T + Gumbel noise) draws from
softmax(logits/T), top-k keeps the k largest and ties at the threshold, keys give independent streams."""

import numpy as np

from tests.plain import sampling as plain


def test_uniforms_are_reproducible_open_and_key_dependent():
    a = plain.uniforms(42, 3, 5, 1000)
    assert a.dtype == np.float32 and np.array_equal(a, plain.uniforms(42, 3, 5, 1000))
    assert a.min() > 0 and a.max() < 1 and 0.45 < a.mean() < 0.55
    for other in (plain.uniforms(43, 3, 5, 1000), plain.uniforms(42, 4, 5, 1000), plain.uniforms(42, 3, 6, 1000)):
        assert abs(np.corrcoef(a, other)[0, 1]) < 0.1
    # one known value pins the generator: a change of constants or shifts is caught
    x = (42 * 0x9E3779B97F4A7C15 + 3 * 0xBF58476D1CE4E5B9 + 5 * 0x94D049BB133111EB + 7) % 2**64
    x ^= x >> 30; x = x * 0xBF58476D1CE4E5B9 % 2**64
    x ^= x >> 27; x = x * 0x94D049BB133111EB % 2**64
    x ^= x >> 31
    assert a[7] == np.float32(((x >> 41) + 0.5) / 8388608.0)


def test_greedy_and_top_k_rules():
    logits = np.array([0.1, 2.0, 2.0, -1.0, 1.5], dtype=np.float32)
    assert plain.sample(logits, 0, None, 0, 0, 0) == 1  # lowest index wins the tie
    assert plain.top_k_mask(logits, 2).tolist() == [False, True, True, False, False]
    assert plain.top_k_mask(logits, 3).tolist() == [False, True, True, False, True]
    tie = np.array([1.0, 3.0, 2.0, 2.0], dtype=np.float32)
    assert plain.top_k_mask(tie, 2).tolist() == [False, True, True, True]  # ties at the threshold survive
    assert plain.top_k_mask(logits, None).all() and plain.top_k_mask(logits, 99).all()


def test_draws_follow_the_softmax():
    logits = np.array([1.0, 0.0, -1.0, 2.0, 0.5], dtype=np.float32)
    for temperature, top_k in ((0.8, None), (1.5, 3)):
        z = logits / temperature
        keep = plain.top_k_mask(logits, top_k)
        p = np.where(keep, np.exp(z - z.max()), 0)
        p /= p.sum()
        counts = np.zeros(5)
        n = 20000
        for step in range(n):
            counts[plain.sample(logits, temperature, top_k, seed=1, request=2, step=step)] += 1
        assert np.all(counts[~keep] == 0)
        assert np.abs(counts / n - p).max() < 0.015

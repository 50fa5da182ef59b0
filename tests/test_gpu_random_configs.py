"""The engine against the plain implementation on configurations and schedules drawn from a seed: head sizes in steps
of 8 from 8 to 256, one to eight kv heads with groups of 1 to 16, widths and feed-forward widths that are no power of
two and no product of the head sizes, one to three layers, odd vocabularies, tied and untied heads, three values of the
norms' eps and of the rotary base; batches of one to eleven requests whose prompts end on, before and after the edges
of a cache page, whose continuations are decoded one token a step for 0 to 70 steps (a request that is through leaves
its batch), and a second batch that takes the first one's slots.  Every page starts as NaN.

What a configuration allows must either run right or be refused; this draws what the fixed tiny configurations do not
reach (a head size of 40 or 136, a group of 7 with one kv head, a width of 2,056).  Tolerances are those of the other
tests: float32 within 1e-4 of the float64 oracle; bfloat16 at most twice the error of the plain implementation with
bfloat16 matrix products (the reference's rule for a low-precision kernel, tests/test_flash_attention_2.py:54-58).
"""

import random
import tempfile

import pytest
import torch

from tests.plain import model as plain
from tests.plain.weights import read_safetensors

pytestmark = pytest.mark.gpu

LENGTHS = [1, 2, 3, 15, 16, 17, 31, 33, 63, 64, 65, 100, 127, 128, 129, 191, 200, 255, 256, 257, 300, 400, 513, 640, 777]


def drawn_config(rng: random.Random) -> dict:
    n_kv = rng.choice([1, 2, 3, 4, 8])
    group = rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 16] if n_kv <= 2 else [1, 2, 3, 4, 8])
    return {
        "arch": "transformer", "vocab_size": rng.choice([100, 257, 1000, 5003]),
        "hidden_size": rng.choice([40, 72, 136, 264, 520, 776, 1032, 1024, 2056]),
        "intermediate_size": rng.choice([88, 200, 328, 1000, 1544, 3080]),
        "num_hidden_layers": rng.choice([1, 2, 3]), "num_attention_heads": n_kv * group, "num_key_value_heads": n_kv,
        "head_dim": rng.choice([8, 16, 24, 32, 40, 48, 64, 72, 80, 96, 112, 128, 136, 160, 192, 256]),
        "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-4]), "rope_theta": rng.choice([1e4, 1e5, 1e6]),
        "tie_word_embeddings": rng.random() < 0.5, "initializer_range": 0.02, "max_position_embeddings": 1024,
    }


def oracle_and_yardstick(tokens, weights, cfg, with_yardstick):
    ids = torch.tensor(tokens, device="cuda")
    oracle = plain.forward(ids, weights, cfg, torch.float64)
    if not with_yardstick:
        return oracle, 0.0
    plain.LOWP = torch.bfloat16
    try:
        low = plain.forward(ids, weights, cfg, torch.float32).double()
    finally:
        plain.LOWP = None
    return oracle, (low - oracle).abs().max().item()


@pytest.mark.parametrize("seed", [3, 11, 23, 42, 57, 64, 78, 91, 105, 117])
def test_drawn_configuration_and_schedule(seed):
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    rng = random.Random(seed)
    cfg = drawn_config(rng)
    n_req = rng.choice([1, 2, 3, 5, 8, 11])
    batches = [([rng.choice(LENGTHS) for _ in range(n_req)], [rng.choice([0, 1, 2, 5, 33, 70]) for _ in range(n_req)])
               for _ in range(2)]
    room = max(sum(-(-(n + d) // 64) * 64 for n, d in zip(*batch)) for batch in batches)  # one batch at a time
    what = f"seed {seed}: {cfg}, prompts and decoded tokens {batches}"
    with tempfile.TemporaryDirectory(prefix="gtar_test_drawn_") as folder:
        # logits of size O(1) whatever the width, so that an error of 1e-3 is an error
        write_random_model(folder, config_from_dict(cfg), seed=seed, std=min(0.08, 0.9 / cfg["hidden_size"] ** 0.5))
        weights = {name: t.cuda() for name, t in read_safetensors(folder + "/model.safetensors").items()}
        for dtype in ("float32", "bfloat16"):
            engine = Engine(load(folder, dtype, "cuda:0"), room, max_seqs=n_req)
            for group in engine.cache.kv_groups:
                group.k.fill_(float("nan"))
                group.v.fill_(float("nan"))
            for number, (prompts, decoded) in enumerate(batches):
                gen = torch.Generator().manual_seed(seed * 10 + number)
                requests = [torch.randint(0, cfg["vocab_size"], (n + d,), generator=gen).tolist()
                            for n, d in zip(prompts, decoded)]
                checked = [oracle_and_yardstick(tokens, weights, cfg, dtype == "bfloat16") for tokens in requests]
                limit = 1e-4 if dtype == "float32" else 2 * max(y for _, y in checked) + 1e-4
                wants = [sorted({n - 1, rng.randrange(n), rng.randrange(n)}) for n in prompts]
                got = engine.step([StepEntry(i, requests[i][:prompts[i]], wants[i]) for i in range(n_req)]).double()
                row = 0
                for i in range(n_req):
                    for place in wants[i]:
                        err = (got[row] - checked[i][0][place]).abs().max().item()
                        assert err < limit, f"{what}\n{dtype} batch {number} request {i} place {place} of its prompt: {err:.3e} (limit {limit:.3e})"
                        row += 1
                engine.end([i for i in range(n_req) if decoded[i] == 0])
                live = [i for i in range(n_req) if decoded[i] > 0]
                step = 0
                while live:
                    got = engine.step([StepEntry(i, [requests[i][prompts[i] + step]], [0]) for i in live]).double()
                    for row, i in enumerate(live):
                        err = (got[row] - checked[i][0][prompts[i] + step]).abs().max().item()
                        assert err < limit, f"{what}\n{dtype} batch {number} request {i} decoded token {step}: {err:.3e} (limit {limit:.3e})"
                    step += 1
                    engine.end([i for i in live if decoded[i] == step])
                    live = [i for i in live if decoded[i] > step]
            del engine

"""Generation through the Python entry point and the command line: greedy tokens against the
plain implementation, long decoding, the first tokens of a sequence, stop tokens, seeded
temperature sampling against the plain sampler, and independence from the batch."""

import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.helpers import CONFIGS, check_against_plain, load_engine, model_folder, plain_logits, requests_for
from tests.plain import sampling as plain_sampling

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def api():
    from gtar_kimik3_public_b200 import generate

    return generate


def plain_greedy(tag, prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        token = int(plain_logits(tag, ids, "f64")[-1].argmax())
        out.append(token)
        ids.append(token)
    return out


@pytest.mark.parametrize("tag", ["tiny_a", "tiny_b"])
def test_greedy_generation_float32_equals_plain(tag):
    model = api().load(model_folder(tag), "float32")
    prompts = requests_for(tag, [5, 17, 32, 1], seed=21)
    got = api().generate(model, prompts, max_new_tokens=16, temperature=0.0)
    for prompt, tokens in zip(prompts, got):
        assert tokens == plain_greedy(tag, prompt, 16)


@pytest.mark.parametrize("tag", ["tiny_a", "tiny_b"])
def test_greedy_generation_bfloat16_picks_a_top_token(tag):
    model = api().load(model_folder(tag), "bfloat16")
    prompts = requests_for(tag, [5, 17, 32, 1], seed=21)
    got = api().generate(model, prompts, max_new_tokens=16, temperature=0.0)
    for prompt, tokens in zip(prompts, got):
        assert len(tokens) == 16
        ids = list(prompt)
        for token in tokens:
            oracle = plain_logits(tag, ids, "f64")[-1]
            lowp = plain_logits(tag, ids, "lowp")[-1].double()
            slack = 2 * (2 * (lowp - oracle).abs().max().item() + 1e-4)  # both candidates may be off by the bound
            assert oracle[token] >= oracle.max() - slack, "bfloat16 greedy chose a token that is not near the top"
            ids.append(token)


def test_long_decoding_float32():
    tag = "tiny_b"  # context 256: a prompt of 6 and 250 new tokens fill it to the last place
    model = api().load(model_folder(tag), "float32")
    prompt = requests_for(tag, [6], seed=22)[0]
    got = api().generate(model, [prompt], max_new_tokens=250, temperature=0.0)[0]
    assert got == plain_greedy(tag, prompt, 250)
    # asking for more than the context holds ends at the context's end
    more = api().generate(model, [prompt], max_new_tokens=400, temperature=0.0)[0]
    assert len(more) == 256 - 6 + 1 and more[:250] == got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence_one_by_one(dtype):
    from gtar_kimik3_public_b200.engine import StepEntry

    tag = "tiny_a"
    engine = load_engine(tag, dtype, max_tokens=128)
    tokens = requests_for(tag, [4], seed=23)[0]
    rows = [engine.step([StepEntry("r", [t], [0])]) for t in tokens]  # position 0 alone, then 1, 2, 3
    check_against_plain(tag, dtype, tokens, [0, 1, 2, 3], torch.cat(rows), "first tokens one by one")
    engine.end(["r"])


def test_stop_token_ends_a_sequence_and_is_emitted():
    tag = "tiny_a"
    model = api().load(model_folder(tag), "float32")
    prompts = requests_for(tag, [9, 12], seed=24)
    free_run = api().generate(model, prompts, max_new_tokens=12, temperature=0.0)
    stop = free_run[0][4]
    got = api().generate(model, prompts, max_new_tokens=12, temperature=0.0, eos_token_id=stop)
    for free, stopped in zip(free_run, got):
        cut = free.index(stop) + 1 if stop in free else len(free)
        assert stopped == free[:cut]
    assert got[0][-1] == stop and len(got[0]) <= 5


def test_temperature_sampling_matches_the_plain_sampler_and_ignores_the_batch():
    tag, seed, temperature, top_k = "tiny_b", 77, 0.8, 50
    model = api().load(model_folder(tag), "float32")
    prompts = requests_for(tag, [1, 9, 40, 64], seed=25)
    got = api().generate(model, prompts, max_new_tokens=24, temperature=temperature, top_k=top_k, seed=seed)
    again = api().generate(model, prompts, max_new_tokens=24, temperature=temperature, top_k=top_k, seed=seed)
    other = api().generate(model, prompts, max_new_tokens=24, temperature=temperature, top_k=top_k, seed=seed + 1)
    assert got == again and got != other
    for r, (prompt, tokens) in enumerate(zip(prompts, got)):
        ids = list(prompt)
        for step, token in enumerate(tokens):
            logits = plain_logits(tag, ids, "f32")[-1].numpy()
            assert token == plain_sampling.sample(logits, temperature, top_k, seed, r, step), (r, step)
            ids.append(token)
    # a request alone in its batch draws the same tokens as in the batch of four
    generator = api().Generator(model, max_tokens=4 * 128, max_batch=1)
    alone = generator.generate(prompts, max_new_tokens=24, temperature=temperature, top_k=top_k, seed=seed)
    assert alone == got


def test_more_requests_than_the_cache_holds_at_once():
    tag = "tiny_a"
    model = api().load(model_folder(tag), "float32")
    prompts = requests_for(tag, [3, 50, 7, 64, 20, 1, 33, 90], seed=26)
    generator = api().Generator(model, max_tokens=256, max_batch=3)  # at most three at a time, 256 tokens in all
    got = generator.generate(prompts, max_new_tokens=10, temperature=0.0)
    for prompt, tokens in zip(prompts, got):
        assert tokens == plain_greedy(tag, prompt, 10)
    assert generator.engine.cache.slots.n_used == 0


def test_command_line(tmp_path):
    tag = "tiny_a"
    prompts = requests_for(tag, [5, 11], seed=27)
    arg = ";".join(",".join(str(t) for t in p) for p in prompts)
    cmd = [sys.executable, "-m", "gtar_kimik3_public_b200.scripts.generate", "--model", str(model_folder(tag)), "--dtype",
           "float32", "--prompt-ids", arg, "--max-new-tokens", "6", "--temperature", "0"]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [line for line in out.stdout.splitlines() if line and line != "---"]
    assert [[int(t) for t in line.split(",")] for line in lines] == [plain_greedy(tag, p, 6) for p in prompts]


def test_generator_sizes_its_cache_itself():
    """Without ``max_tokens`` the generator takes room for ``max_batch`` sequences of the longest context the
    configuration allows, but no more than fits in most of the free device memory."""
    tag = "tiny_b"
    model = api().load(model_folder(tag), "float32")
    generator = api().Generator(model, max_batch=5)
    assert generator.engine.cache.n_pages * generator.engine.cache.page_size == 5 * 256
    wanted = api().Generator.default_max_tokens(model, 5)
    assert wanted == 5 * 256
    free, _ = torch.cuda.mem_get_info()
    per_token = generator.engine.cache.kv_bytes_per_token()
    little = 200 * per_token / free  # a device with room for 200 tokens: three pages
    assert api().Generator.default_max_tokens(model, 5, share_of_free_memory=little) == 192
    with pytest.raises(RuntimeError, match="no device memory"):
        api().Generator.default_max_tokens(model, 5, share_of_free_memory=little / 100)
    prompts = requests_for(tag, [4, 30], seed=28)
    got = generator.generate(prompts, max_new_tokens=5, temperature=0.0)
    assert got == [plain_greedy(tag, p, 5) for p in prompts]


def test_weights_drawn_on_the_device():
    """The random-weights mode without a folder (the benchmark's 4B and 8B points): types as the loader's rule gives
    them, a fixed seed gives the same model, and the model steps."""
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.models.model import Model
    from gtar_kimik3_public_b200.registry import architecture, config_from_dict
    from gtar_kimik3_public_b200.weights import load_random_weights
    from tests.helpers import CONFIGS

    config = config_from_dict(CONFIGS["tiny_c"])
    logits = []
    for seed in (3, 3, 4):
        model = Model(architecture(config.ARCH_NAMES[0]).build_plan(config), config, torch.bfloat16, "cuda:0")
        load_random_weights(model, seed=seed, std=0.08)
        layer = model.plan.layers[0]
        assert layer.mixer.w_qkv.dtype == torch.bfloat16 and layer.input_norm.weight.dtype == torch.float32
        engine = Engine(model, 128, max_seqs=1)
        logits.append(engine.step([StepEntry("r", list(range(1, 40)), [38])]))
    assert torch.isfinite(logits[0]).all() and logits[0].abs().max() > 0.1
    assert torch.equal(logits[0], logits[1]) and not torch.equal(logits[0], logits[2])


def test_command_line_takes_a_checkpoint_of_the_reference(tmp_path):
    """``--checkpoint FILE`` as in the reference's command line (scripts/generate.py:19-20,33-37): converted to a model
    folder first; the greedy tokens are those stored under tests/golden/."""
    import numpy as np

    from tests.test_convert import GOLDEN, write_checkpoint
    from tests.tiny_configs import TINY_A

    write_checkpoint(tmp_path / "ckpt.pt", TINY_A, 0)
    data = np.load(GOLDEN / "tiny_a.npz")
    prompts = [data[f"ids_{r}"].tolist() for r in range(3)]
    want = [data[f"greedy_{r}"].tolist() for r in range(3)]
    arg = ";".join(",".join(str(t) for t in p) for p in prompts)
    cmd = [sys.executable, "-m", "gtar_kimik3_public_b200.scripts.generate", "--checkpoint", str(tmp_path / "ckpt.pt"), "--dtype",
           "float32", "--prompt-ids", arg, "--max-new-tokens", str(len(want[0])), "--temperature", "0"]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [line for line in out.stdout.splitlines() if line and line != "---"]
    assert [[int(t) for t in line.split(",")] for line in lines] == want

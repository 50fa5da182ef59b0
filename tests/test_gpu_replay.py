"""The engine against the plain implementation under every way of cutting the work: each request
alone and whole; with its last 32 tokens one by one; in batches of unequal lengths whose shorter
requests end earlier, one batch after another on a cache too small for all of them at once, so
that slots and pages are used again.  In float32 and in bfloat16, for both tiny configurations."""

import pytest
import torch

from tests.helpers import CONFIGS, check_against_plain, load_engine, poison, requests_for

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [1, 5, 33, 64, 65, 100, 128], "tiny_b": [1, 9, 40, 64, 129, 200, 256],
           "tiny_c": [1, 31, 64, 130, 257, 400, 512]}
CASES = [(tag, dtype) for tag in ("tiny_a", "tiny_b", "tiny_c") for dtype in ("float32", "bfloat16")]


def _entry(request_id, tokens, want):
    from gtar_kimik3_public_b200.engine import StepEntry

    return StepEntry(request_id, tokens, want)


@pytest.mark.parametrize("tag,dtype", CASES)
def test_each_request_alone_and_whole(tag, dtype):
    engine = load_engine(tag, dtype, max_tokens=512)
    poison(engine)
    for r, tokens in enumerate(requests_for(tag, LENGTHS[tag])):
        places = list(range(len(tokens)))
        logits = engine.step([_entry(r, tokens, places)])
        engine.end([r])
        assert logits.shape == (len(tokens), CONFIGS[tag]["vocab_size"])
        check_against_plain(tag, dtype, tokens, places, logits, f"{tag} {dtype} request {r} whole")
        engine.cache.check_invariants()
    assert engine.cache.slots.n_used == 0


@pytest.mark.parametrize("tag,dtype", CASES)
def test_last_32_tokens_one_by_one(tag, dtype):
    engine = load_engine(tag, dtype, max_tokens=512)
    poison(engine)
    for r, tokens in enumerate(requests_for(tag, LENGTHS[tag])):
        if len(tokens) <= 32:
            continue
        head = len(tokens) - 32
        whole = engine.step([_entry(("w", r), tokens, list(range(len(tokens))))])
        engine.end([("w", r)])
        parts = [engine.step([_entry(r, tokens[:head], list(range(head)))])]
        for t in range(head, len(tokens)):
            parts.append(engine.step([_entry(r, [tokens[t]], [0])]))
        engine.end([r])
        stepped = torch.cat(parts)
        check_against_plain(tag, dtype, tokens, list(range(len(tokens))), stepped, f"{tag} {dtype} request {r} stepped")
        if dtype == "float32":
            # the 32-bit kernels reduce in an order that does not depend on the cut: bit-equal
            assert torch.equal(stepped, whole), f"{tag} request {r}: stepping changed float32 logits"


@pytest.mark.parametrize("tag,dtype", CASES)
def test_unequal_batches_with_slot_reuse(tag, dtype):
    requests = requests_for(tag, LENGTHS[tag] + LENGTHS[tag][::-1], seed=11)
    longest = max(len(t) for t in requests)
    # room for three of the longest requests only: batches of three, one after another
    engine = load_engine(tag, dtype, max_tokens=3 * (-(-longest // 64) * 64), max_seqs=3)
    poison(engine)
    alone = {}
    if dtype == "float32":
        for r, tokens in enumerate(requests):
            alone[r] = engine.step([_entry(("a", r), tokens, list(range(len(tokens))))])
            engine.end([("a", r)])
    for start in range(0, len(requests), 3):
        batch = list(range(start, min(start + 3, len(requests))))
        # prompts: all but the last (up to) 8 tokens of each request, in one step
        prompt_len = {r: max(1, len(requests[r]) - 8) for r in batch}
        got = {r: [] for r in batch}
        logits = engine.step([_entry(r, requests[r][:prompt_len[r]], list(range(prompt_len[r]))) for r in batch])
        offset = 0
        for r in batch:
            got[r].append(logits[offset:offset + prompt_len[r]])
            offset += prompt_len[r]
        fed = dict(prompt_len)
        live = [r for r in batch if fed[r] < len(requests[r])]
        done = [r for r in batch if r not in live]
        if done:
            engine.end(done)
        while live:
            logits = engine.step([_entry(r, [requests[r][fed[r]]], [0]) for r in live])
            for i, r in enumerate(live):
                got[r].append(logits[i:i + 1])
                fed[r] += 1
            done = [r for r in live if fed[r] == len(requests[r])]
            if done:
                engine.end(done)  # the shorter requests end earlier; the others go on
            live = [r for r in live if r not in done]
            engine.cache.check_invariants()
        for r in batch:
            tokens = requests[r]
            stacked = torch.cat(got[r])
            check_against_plain(tag, dtype, tokens, list(range(len(tokens))), stacked, f"{tag} {dtype} request {r} batched")
            if dtype == "float32":
                assert torch.equal(stacked, alone[r]), f"{tag} request {r}: batching changed float32 logits"
    assert engine.cache.slots.n_used == 0
    assert all(g.pages.n_used == 0 for g in engine.cache.kv_groups)


@pytest.mark.parametrize("tag,dtype", CASES)
def test_wanted_places_subset_and_empty(tag, dtype):
    engine = load_engine(tag, dtype, max_tokens=512)
    a, b = requests_for(tag, [50, 70], seed=3)
    logits = engine.step([_entry("a", a, [0, 49]), _entry("b", b, [])])
    assert logits.shape[0] == 2
    check_against_plain(tag, dtype, a, [0, 49], logits, "subset of places")
    # b was cached although nothing was asked of it
    nxt = engine.step([_entry("a", [a[0]], []), _entry("b", [b[0]], [0])])
    check_against_plain(tag, dtype, b + [b[0]], [70], nxt, "continuation after a step without wanted places")
    engine.end(["a", "b"])


@pytest.mark.parametrize("tag,dtype", CASES)
def test_replayed_graph_steps_equal_plain_launches(tag, dtype):
    """Decode steps run from a captured CUDA graph give the very numbers of kernels launched one by one."""
    requests = requests_for(tag, [70, 3, 64], seed=13)
    results = []
    for use_graphs in (False, True):
        engine = load_engine(tag, dtype, max_tokens=3 * 128, max_seqs=3, use_graphs=use_graphs)
        assert (engine.graphs is not None) == use_graphs
        poison(engine)
        engine.step([_entry(r, requests[r][:-20] or requests[r][:1], []) for r in range(3)])
        fed = {r: max(1, len(requests[r]) - 20) for r in range(3)}
        rows = []
        live = [0, 1, 2]
        while live:
            rows.append(engine.step([_entry(r, [requests[r][fed[r]]], [0]) for r in live]))
            for r in live:
                fed[r] += 1
            done = [r for r in live if fed[r] == len(requests[r])]
            engine.end(done)
            live = [r for r in live if r not in done]
        results.append(torch.cat(rows))
    assert torch.equal(results[0], results[1])


@pytest.mark.parametrize("tag,dtype,n_requests", [("tiny_a", "bfloat16", 13), ("tiny_b", "bfloat16", 16), ("tiny_c", "bfloat16", 20),
                                                  ("tiny_b", "float32", 13)])
def test_decode_in_batches_of_more_than_eight(tag, dtype, n_requests):
    """Nine to sixteen sequences take other kernel variants than a handful (two row blocks in the few-token
    product), seventeen and more the many-token product: prompts of unequal lengths in one step, then eight
    tokens each, the shorter requests ending earlier."""
    lengths = [10 + (7 * i) % 60 for i in range(n_requests)]
    requests = requests_for(tag, lengths, seed=23)
    engine = load_engine(tag, dtype, max_tokens=n_requests * 128, max_seqs=n_requests)
    poison(engine)
    batch = list(range(n_requests))
    prompt_len = {r: max(1, len(requests[r]) - 8 + (r % 3)) for r in batch}  # 6 to 8 tokens left to decode
    got = {r: [] for r in batch}
    logits = engine.step([_entry(r, requests[r][:prompt_len[r]], list(range(prompt_len[r]))) for r in batch])
    offset = 0
    for r in batch:
        got[r].append(logits[offset:offset + prompt_len[r]])
        offset += prompt_len[r]
    fed = dict(prompt_len)
    live = list(batch)
    while live:
        logits = engine.step([_entry(r, [requests[r][fed[r]]], [0]) for r in live])
        for i, r in enumerate(live):
            got[r].append(logits[i:i + 1])
            fed[r] += 1
        done = [r for r in live if fed[r] == len(requests[r])]
        if done:
            engine.end(done)
        live = [r for r in live if r not in done]
    for r in batch:
        tokens = requests[r]
        check_against_plain(tag, dtype, tokens, list(range(len(tokens))), torch.cat(got[r]), f"{tag} {dtype} request {r} of {n_requests}")
    assert engine.cache.slots.n_used == 0


@pytest.mark.parametrize("cast", [False, True])
def test_folder_stored_in_32_bit_run_in_bfloat16(tmp_path, cast):
    """A folder whose matrices are stored in 32-bit, run in bfloat16.  By default a tensor stored in 32-bit stays
    so: its projections run on the exact 32-bit kernel (the loader warns that this is slow) and the logits are
    closer to the oracle than bfloat16 weights could make them.  With ``cast_matrices`` the matrices are rounded
    to bfloat16 at load, as the reference's autocast rounds them at every projection (src/engine.py:35), and the
    model is the same as one loaded from the rounded folder."""
    import warnings

    from gtar_kimik3_public_b200.engine import Engine
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model
    from tests.plain import model as plain
    from tests.plain.weights import read_safetensors

    cfg = CONFIGS["tiny_b"]
    folder = write_random_model(tmp_path / "f32", config_from_dict(cfg), seed=5, std=0.08, matrix_dtype=torch.float32)
    weights = read_safetensors(folder / "model.safetensors")
    assert weights["model.layers.0.mlp.down_proj.weight"].dtype == torch.float32
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        model = load(folder, "bfloat16", "cuda:0", cast_matrices=cast)
    assert any("32-bit" in str(w.message) for w in caught) == (not cast)
    kept = model.plan.layers[0].feed_forward.w_down.dtype
    assert kept == (torch.bfloat16 if cast else torch.float32)
    engine = Engine(model, 256, max_seqs=2)
    (tokens,) = requests_for("tiny_b", [90], seed=5)
    head = len(tokens) - 10
    parts = [engine.step([_entry("r", tokens[:head], list(range(head)))])]
    for t in range(head, len(tokens)):
        parts.append(engine.step([_entry("r", [tokens[t]], [0])]))
    got = torch.cat(parts).double().cpu()
    if cast:
        weights = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in weights.items()}
    oracle = plain.forward(torch.tensor(tokens), weights, cfg, torch.float64)
    plain.LOWP = torch.bfloat16
    try:
        lowp = plain.forward(torch.tensor(tokens), weights, cfg, torch.float32).double()
    finally:
        plain.LOWP = None
    err, yard = (got - oracle).abs().max().item(), (lowp - oracle).abs().max().item()
    assert err <= 2 * yard + 1e-4, f"error {err:.3e} against a yardstick of {yard:.3e}"

"""The engine against the plain implementation at the layer sizes of the benchmark configurations (Qwen3-0.6B, 4B and
8B sizes: head size 128, widths 1,024 / 2,560 / 4,096), with few layers and a small vocabulary.  At these sizes a
step takes the kernels that the benchmark times, and none of the tiny configurations reaches them: the q|k|v product
with norm, rotation and cache write in its output stage, the tcgen05 prefill attention, the persistent and paired
many-token products and the library product, decode attention at head size 128 fused with the q/k preparation, the
few-token products and, from 17 and 33 sequences on, the swap-AB tensor-memory products with split K.

Schedules: a long prompt whole; its last 32 tokens one by one (from CUDA graphs); batches of unequal lengths whose
shorter requests end earlier, one batch after another on a cache that holds one batch only; many-token steps replayed
from a graph with the same shape and another split of the tokens among the sequences; decode steps of 40 and 64
sequences.  float32: bit-equal across cuts and within 1e-4 of the float64 oracle.  bfloat16: the reference's rule
(tests/test_flash_attention_2.py:54-58): at most twice the error of a standard low-precision implementation.
Shaped after the reference's own check of cached against whole-prompt logits (tests/test_inference.py:17-38).
"""

import pytest
import torch

from tests.helpers import CONFIGS, check_against_plain, load_engine, poison, requests_for

pytestmark = pytest.mark.gpu

CASES = [("real_06b", "bfloat16"), ("real_06b", "float32"), ("real_4b", "bfloat16"), ("real_4b", "float32"),
         ("real_8b", "bfloat16"), ("real_8b", "float32")]
LONG = {"real_06b": 1800, "real_4b": 1300, "real_8b": 1300}  # enough for 200 tiles of 128 x 256 in the q|k|v product


def _entry(request_id, tokens, want):
    from gtar_kimik3_public_b200.engine import StepEntry

    return StepEntry(request_id, tokens, want)


@pytest.fixture
def kernel_log(monkeypatch):
    """Names of the library's kernels entered while the test runs (launched or captured)."""
    from gtar_kimik3_public_b200.ops import functional as F

    names = []
    real = F.call

    def recording_call(name, *args):
        names.append(name)
        return real(name, *args)

    monkeypatch.setattr(F, "call", recording_call)
    return names


@pytest.mark.parametrize("tag,dtype", CASES)
def test_long_prompt_whole_and_last_32_one_by_one(tag, dtype, kernel_log):
    n = LONG[tag]
    engine = load_engine(tag, dtype, max_tokens=2048, max_seqs=2)
    poison(engine)
    (tokens,) = requests_for(tag, [n], seed=31)
    places = list(range(n))
    whole = engine.step([_entry("whole", tokens, places)])
    engine.end(["whole"])
    assert whole.shape == (n, CONFIGS[tag]["vocab_size"])
    check_against_plain(tag, dtype, tokens, places, whole, f"{tag} {dtype} whole")
    if dtype == "bfloat16":  # the paths that the benchmark times did run
        assert "gk_gemm_bf16_tc_qkv" in kernel_log, "the q|k|v product did not take its fused output stage"
        assert "gk_attention_prefill_tc_tokens_bf16" in kernel_log, "prefill attention did not take the tcgen05 kernel"
    del kernel_log[:]
    head = n - 32
    parts = [engine.step([_entry("cut", tokens[:head], list(range(head)))])]
    for t in range(head, n):
        parts.append(engine.step([_entry("cut", [tokens[t]], [0])]))
    engine.end(["cut"])
    stepped = torch.cat(parts)
    check_against_plain(tag, dtype, tokens, places, stepped, f"{tag} {dtype} last 32 one by one")
    if dtype == "float32":
        assert torch.equal(stepped, whole), f"{tag}: stepping changed float32 logits"
    else:
        assert "gk_attention_decode_fused_bf16" in kernel_log, "decode did not take the fused attention kernel"
        assert "gk_gemv_bf16" in kernel_log, "decode did not take the few-token product"
    assert engine.graphs is not None and len(engine.graphs.graphs) >= 1
    engine.check()
    engine.cache.check_invariants()


@pytest.mark.parametrize("tag,dtype", CASES[:4])
def test_unequal_batches_with_slot_reuse(tag, dtype):
    longest = LONG[tag]
    lengths = [longest, 300, 1, 65, 64, 129, longest - 257, 2]
    requests = requests_for(tag, lengths, seed=37)
    room = sum(-(-n // 64) * 64 for n in lengths[:4])
    engine = load_engine(tag, dtype, max_tokens=room, max_seqs=4)  # one batch fills the cache: the next uses it again
    poison(engine)
    alone = {}
    if dtype == "float32":
        for r, tokens in enumerate(requests):
            alone[r] = engine.step([_entry(("a", r), tokens, list(range(len(tokens))))])
            engine.end([("a", r)])
    for start in (0, 4):
        batch = list(range(start, start + 4))
        prompt_len = {r: max(1, len(requests[r]) - 8) for r in batch}
        got = {r: [] for r in batch}
        logits = engine.step([_entry(r, requests[r][:prompt_len[r]], list(range(prompt_len[r]))) for r in batch])
        offset = 0
        for r in batch:
            got[r].append(logits[offset:offset + prompt_len[r]])
            offset += prompt_len[r]
        fed = dict(prompt_len)
        live = [r for r in batch if fed[r] < len(requests[r])]
        engine.end([r for r in batch if r not in live])
        while live:
            logits = engine.step([_entry(r, [requests[r][fed[r]]], [0]) for r in live])
            for i, r in enumerate(live):
                got[r].append(logits[i:i + 1])
                fed[r] += 1
            done = [r for r in live if fed[r] == len(requests[r])]
            engine.end(done)
            live = [r for r in live if r not in done]
            engine.cache.check_invariants()
        for r in batch:
            tokens = requests[r]
            stacked = torch.cat(got[r])
            check_against_plain(tag, dtype, tokens, list(range(len(tokens))), stacked, f"{tag} {dtype} request {r} batched")
            if dtype == "float32":
                assert torch.equal(stacked, alone[r]), f"{tag} request {r}: batching changed float32 logits"
    assert engine.cache.slots.n_used == 0
    engine.check()


@pytest.mark.parametrize("tag,dtype", [("real_06b", "bfloat16"), ("tiny_c", "bfloat16"), ("tiny_c", "float32")])
def test_many_token_graph_serves_another_split_of_the_same_shape(tag, dtype):
    """A step of several tokens per sequence is captured when its shape comes a second time and replayed from then
    on.  The shape is (tokens, sequences, wanted rows, longest part): 100/60/40 tokens and 100/50/50 tokens share it,
    and a launch that had baked the first split in at capture would give the second split wrong numbers."""
    scale = 17 if tag == "real_06b" else 1  # 1,700 / 1,020 / 680 tokens at the real sizes
    splits = [(100, 60, 40), (100, 60, 40), (100, 50, 50), (100, 40, 60), (100, 99, 1)]
    engine = load_engine(tag, dtype, max_tokens=3 * 2048 if scale > 1 else 512, max_seqs=3)
    poison(engine)
    assert engine.graphs is not None
    for round_index, split in enumerate(splits):
        lengths = [n * scale for n in split]
        requests = requests_for(tag, lengths, seed=41 + round_index)
        wanted = [[0, n // 2, n - 1] for n in lengths]  # three rows each: the same number of wanted rows every round
        logits = engine.step([_entry(r, requests[r], wanted[r]) for r in range(3)])
        for r in range(3):
            check_against_plain(tag, dtype, requests[r], wanted[r], logits[3 * r:3 * r + 3],
                                f"{tag} {dtype} round {round_index} request {r} of split {split}")
        engine.end([0, 1, 2])
        if round_index >= 1:
            assert any(key[3] == 100 * scale for key in engine.graphs.graphs), "the many-token shape was not captured"
    engine.check()


@pytest.mark.parametrize("tag,dtype,n_requests", [("real_06b", "bfloat16", 12), ("real_06b", "bfloat16", 40), ("real_06b", "bfloat16", 64), ("real_4b", "bfloat16", 33),
                                                  ("tiny_c", "bfloat16", 40), ("tiny_a", "bfloat16", 64), ("real_06b", "float32", 40)])
def test_decode_steps_of_many_sequences(tag, dtype, n_requests, kernel_log):
    """33 to 64 sequences: every product of a decode step runs in the swap-AB orientation on tcgen05, with K split
    among the blocks of a cluster where K is long enough (the real sizes)."""
    expect = []
    if dtype == "bfloat16":
        # 9 to 32 sequences: the few-token product and decode attention fused with the q/k preparation
        expect = ["gk_gemm_bf16_tc"] if n_requests > 32 else ["gk_gemv_bf16", "gk_attention_decode_fused_bf16"]
    _decode_many(tag, dtype, n_requests, kernel_log, expect)


@pytest.mark.parametrize("tag,n_requests", [("real_06b", 12), ("real_06b", 40), ("real_4b", 33), ("tiny_c", 40), ("tiny_c", 3)])
def test_decode_steps_with_the_pages_dealt_evenly(tag, n_requests, kernel_log, monkeypatch):
    """The decode attention kernel that cuts the line of all sequences' pages into equal pieces, forced for every
    step: sequences of unequal lengths that end one after another, inside captured steps."""
    from gtar_kimik3_public_b200.ops import attention as attention_ops

    monkeypatch.setattr(attention_ops, "DECODE_FLAT", "always")
    _decode_many(tag, "bfloat16", n_requests, kernel_log, ["gk_attention_decode_flat_bf16"])
    assert "gk_attention_decode_fused_bf16" not in kernel_log and "gk_attention_decode_bf16" not in kernel_log


def test_decode_work_outgrown_by_a_larger_batch_stays_valid_for_captured_steps(monkeypatch):
    """The scratch and the ticket counters of the evenly dealt decode attention belong to the cache group and grow with
    the batch; the captured steps of a smaller batch keep the buffers they were captured with.  Twelve sequences, then
    forty (the buffers grow), then twelve again in the slots given back: all against the plain implementation."""
    from gtar_kimik3_public_b200.ops import attention as attention_ops

    from gtar_kimik3_public_b200.ops.functional import DecodeWork

    monkeypatch.setattr(attention_ops, "DECODE_FLAT", "always")
    monkeypatch.setattr(DecodeWork, "MIN_FLOATS", 1)
    monkeypatch.setattr(DecodeWork, "MIN_PAIRS", 1)
    tag, dtype = "tiny_c", "bfloat16"
    engine = load_engine(tag, dtype, max_tokens=40 * 128, max_seqs=40)
    poison(engine)
    work = None
    for turn, n_requests in enumerate((12, 40, 12)):
        lengths = [5 + (7 * i + turn) % 60 for i in range(n_requests)]
        requests = requests_for(tag, lengths, seed=70 + turn)
        batch = [f"{turn}.{i}" for i in range(n_requests)]
        head = {r: len(t) - 3 for r, t in zip(batch, requests)}
        tokens = dict(zip(batch, requests))
        engine.step([_entry(r, tokens[r][:head[r]], []) for r in batch])
        rows = {r: [] for r in batch}
        for k in range(3):
            logits = engine.step([_entry(r, [tokens[r][head[r] + k]], [0]) for r in batch])
            for i, r in enumerate(batch):
                rows[r].append(logits[i:i + 1])
        engine.end(batch)
        for r in batch:
            check_against_plain(tag, dtype, tokens[r], list(range(head[r], head[r] + 3)), torch.cat(rows[r]), f"turn {turn} request {r}")
        group = engine.cache.kv_groups[0]
        if turn == 0:
            work = group._work
            first_part, first_tickets = work.part, work.tickets
        assert int(group._work.tickets.abs().sum()) == 0
    assert work is engine.cache.kv_groups[0]._work
    assert work.part is not first_part and work.tickets is not first_tickets  # forty sequences outgrew twelve's buffers
    assert any(t is first_part for t in work.outgrown) and int(first_tickets.abs().sum()) == 0
    engine.check()
    assert engine.cache.slots.n_used == 0


def _decode_many(tag, dtype, n_requests, kernel_log, expect):
    lengths = [6 + (11 * i) % 90 for i in range(n_requests)]
    requests = requests_for(tag, lengths, seed=43)
    engine = load_engine(tag, dtype, max_tokens=n_requests * 128, max_seqs=n_requests)
    poison(engine)
    batch = list(range(n_requests))
    prompt_len = {r: max(1, len(requests[r]) - 5 + (r % 3)) for r in batch}  # 3 to 5 tokens left to decode
    got = {r: [] for r in batch}
    logits = engine.step([_entry(r, requests[r][:prompt_len[r]], list(range(prompt_len[r]))) for r in batch])
    offset = 0
    for r in batch:
        got[r].append(logits[offset:offset + prompt_len[r]])
        offset += prompt_len[r]
    fed = dict(prompt_len)
    live = list(batch)
    del kernel_log[:]
    steps = 0
    while live:
        logits = engine.step([_entry(r, [requests[r][fed[r]]], [0]) for r in live])
        if steps == 0:
            for name in expect:
                assert name in kernel_log, f"the first decode step did not call {name}"
        steps += 1
        for i, r in enumerate(live):
            got[r].append(logits[i:i + 1])
            fed[r] += 1
        done = [r for r in live if fed[r] == len(requests[r])]
        engine.end(done)
        live = [r for r in live if r not in done]
    for r in batch:
        tokens = requests[r]
        check_against_plain(tag, dtype, tokens, list(range(len(tokens))), torch.cat(got[r]), f"{tag} {dtype} request {r} of {n_requests}")
    assert engine.cache.slots.n_used == 0
    engine.check()


@pytest.mark.parametrize("n_seqs", [1, 2])
def test_decode_beyond_12288_tokens_merges_its_splits_through_scratch(n_seqs, kernel_log):
    """One and two sequences of more than 12,288 tokens: decode attention cuts each into more pieces than a cluster
    holds, writes partial results to scratch memory and merges them in a second kernel."""
    from gtar_kimik3_public_b200.ops import functional as F

    tag, dtype = "tiny_long", "bfloat16"
    lengths = [12400, 12350][:n_seqs]
    requests = requests_for(tag, lengths, seed=47)
    engine = load_engine(tag, dtype, max_tokens=n_seqs * 12928, max_seqs=n_seqs)
    poison(engine)
    tail = 6
    engine.step([_entry(r, requests[r][:-tail], []) for r in range(n_seqs)])
    del kernel_log[:]
    rows = {r: [] for r in range(n_seqs)}
    for t in range(tail):
        logits = engine.step([_entry(r, [requests[r][len(requests[r]) - tail + t]], [0]) for r in range(n_seqs)])
        for r in range(n_seqs):
            rows[r].append(logits[r:r + 1])
    assert F.decode_splits(n_seqs, 1, 12928, 64, F.sm_count()) > 8
    assert "gk_attention_decode_bf16" in kernel_log and "gk_attention_decode_fused_bf16" not in kernel_log
    for r in range(n_seqs):
        n = len(requests[r])
        check_against_plain(tag, dtype, requests[r], list(range(n - tail, n)), torch.cat(rows[r]), f"sequence {r} beyond 12,288 tokens")
    engine.end(list(range(n_seqs)))
    engine.check()


def test_a_rows_logits_do_not_depend_on_how_many_rows_are_wanted():
    """The output head writes its 32-bit sums whatever the number of wanted rows: a position's logits are not
    rounded to bfloat16 when a step asks for more than a handful of rows (bfloat16 spacing near 1 is 4e-3)."""
    tag, dtype = "real_06b", "bfloat16"
    engine = load_engine(tag, dtype, max_tokens=256, max_seqs=1)
    (tokens,) = requests_for(tag, [200], seed=53)
    one = engine.step([_entry("a", tokens, [150])])
    engine.end(["a"])
    many = engine.step([_entry("b", tokens, list(range(100, 200)))])
    engine.end(["b"])
    assert (one[0] - many[50]).abs().max().item() < 2e-5
    rounded = many.to(torch.bfloat16).to(torch.float32)
    assert (rounded - many).abs().max().item() > 1e-4, "logits look rounded to bfloat16"


@pytest.mark.parametrize("n_seqs", [1, 3, 8])
def test_persistent_kernel_for_all_layers_of_a_decode_step(n_seqs, kernel_log, monkeypatch):
    """The optional path that runs every layer of a small decode step as one persistent kernel (grid-wide barriers
    between a layer's stages, weights and cached keys streamed through per-warp rings across them): unequal
    sequences, the shorter ending earlier, launched one by one and replayed from graphs, over poisoned pages."""
    from gtar_kimik3_public_b200.models import persistent_decode

    monkeypatch.setattr(persistent_decode, "ENABLED", True)
    tag, dtype = "real_06b", "bfloat16"
    requests = requests_for(tag, [70, 3, 200, 64, 65, 129, 17, 300][:n_seqs], seed=59)
    results = []
    for use_graphs in (False, True):
        engine = load_engine(tag, dtype, max_tokens=n_seqs * 512, max_seqs=n_seqs, use_graphs=use_graphs)
        assert engine.model.persistent_decode(engine.cache) is not None
        poison(engine)
        fed = {r: max(1, len(requests[r]) - 6) for r in range(n_seqs)}
        engine.step([_entry(r, requests[r][:fed[r]], []) for r in range(n_seqs)])
        rows = {r: [] for r in range(n_seqs)}
        live = [r for r in range(n_seqs) if fed[r] < len(requests[r])]
        engine.end([r for r in range(n_seqs) if r not in live])
        del kernel_log[:]
        while live:
            logits = engine.step([_entry(r, [requests[r][fed[r]]], [0]) for r in live])
            for i, r in enumerate(live):
                rows[r].append(logits[i:i + 1].clone())
                fed[r] += 1
            done = [r for r in live if fed[r] == len(requests[r])]
            engine.end(done)
            live = [r for r in live if r not in done]
        assert "gk_decode_layers" in kernel_log and "gk_attention_decode_fused_bf16" not in kernel_log
        engine.check()
        for r, got in rows.items():
            if got:
                n = len(requests[r])
                check_against_plain(tag, dtype, requests[r], list(range(n - len(got), n)), torch.cat(got), f"persistent decode, request {r}")
        results.append({r: torch.cat(got) for r, got in rows.items() if got})
    for r in results[0]:
        assert torch.equal(results[0][r], results[1][r]), "replayed from a graph, the persistent kernel gave other numbers"


def test_decode_across_a_bound_on_the_lengths():
    """Decode graphs are keyed by a bound on the longest sequence of the step (1,024, 1,536, 2,048, ...: launches are
    sized from it): a sequence that grows from below 1,024 tokens to above it changes graphs on the way, and its logits
    do not."""
    tag, dtype = "real_06b", "bfloat16"
    (tokens,) = requests_for(tag, [1040], seed=61)
    engine = load_engine(tag, dtype, max_tokens=2048, max_seqs=1)
    poison(engine)
    head = 1010
    engine.step([_entry("r", tokens[:head], [])])
    rows = [engine.step([_entry("r", [tokens[t]], [0])]) for t in range(head, len(tokens))]
    bounds = sorted({key[4] for key in engine.graphs.graphs if key[3] == 1})
    assert bounds == [1024, 1536], bounds
    check_against_plain(tag, dtype, tokens, list(range(head, len(tokens))), torch.cat(rows), "decode across the bound of 1,024 tokens")
    engine.check()

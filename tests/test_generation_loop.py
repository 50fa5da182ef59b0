"""The generation loop's decisions, tested on the CPU with stand-ins for the engine and the
chooser: how requests are batched, what each step is fed, when a sequence ends, that ended
sequences leave at once and their storage is given back, that the last chosen token is not fed."""

from types import SimpleNamespace

import pytest

from gtar_kimik3_public_b200.engine.generation import GenerationParams, form_batches, run_generation


class ScriptedEngine:
    """Counts what the loop asks of an engine.  "Logits" are just the list of (request, fed tokens)."""

    def __init__(self, n_pages=64, page_size=64, max_seq_len=None, max_seqs=8):
        self.cache = SimpleNamespace(n_pages=n_pages, page_size=page_size, max_seq_len=max_seq_len, max_seqs=max_seqs)
        self.slot_of = {}
        self.fed = {}
        self.steps = []
        self.peak_live = 0
        self.ended = []

    def step(self, entries, keep_output=True):
        assert keep_output is False  # the loop consumes the logits at once
        ids = [e.id for e in entries]
        lengths = {len(e.tokens) for e in entries}
        new = [i for i in ids if i not in self.slot_of]
        assert not new or len(new) == len(ids), "a batch's requests start together"
        assert new or lengths == {1}, "after the prompts each live sequence brings one token"
        for e in entries:
            self.slot_of.setdefault(e.id, len(self.slot_of))
            self.fed.setdefault(e.id, []).extend(e.tokens)
            assert e.want == [len(e.tokens) - 1]
        self.peak_live = max(self.peak_live, len(self.slot_of))
        self.steps.append(ids)
        return [(e.id, list(self.fed[e.id])) for e in entries]

    def end(self, ids):
        for i in ids:
            del self.slot_of[i]
            self.ended.append(i)


def chooser_from(plan):
    """``plan[request index]`` is the list of tokens that request will be given, in order."""

    def choose(logits, request_indices, steps):
        assert len(logits) == len(request_indices) == len(steps)
        return [plan[r][s] for r, s in zip(request_indices, steps)]

    return choose


def test_unequal_prompts_stop_tokens_and_early_enders():
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9]]
    plan = {0: [10, 11, 99, 12], 1: [20, 21, 22, 23, 24], 2: [99]}
    engine = ScriptedEngine()
    out = run_generation(engine, prompts, GenerationParams(max_new_tokens=4, stop_ids=frozenset({99})), chooser_from(plan))
    assert out == [[10, 11, 99], [20, 21, 22, 23], [99]]  # the stop token is part of the output
    # request 2 left after the first step, request 0 after the third; request 1 went on alone
    assert [len(s) for s in engine.steps] == [3, 2, 2, 1]
    assert engine.slot_of == {} and len(engine.ended) == 3
    # what was fed: the prompt, then every chosen token but the last
    assert engine.fed[("gen", 0)] == [1, 2, 3, 10, 11]
    assert engine.fed[("gen", 1)] == [4, 20, 21, 22]
    assert engine.fed[("gen", 2)] == [5, 6, 7, 8, 9]


def test_batches_follow_one_another_and_reuse_the_room():
    prompts = [[1] * n for n in (10, 70, 30, 64, 5, 5, 5)]
    plan = {i: [7] * 8 for i in range(len(prompts))}
    engine = ScriptedEngine(n_pages=4, max_seqs=3)
    out = run_generation(engine, prompts, GenerationParams(max_new_tokens=8, max_batch=3), chooser_from(plan))
    assert all(len(o) == 8 for o in out)
    # room is 4 pages of 64 and 3 slots: [10+7 -> 1 page, 70+7 -> 2, 30+7 -> 1], [64+7 -> 2, 5+7 -> 1, 1], [1]
    assert form_batches([len(p) for p in prompts], 8, 3, 256, 64, None, 3) == [[0, 1, 2], [3, 4, 5], [6]]
    assert form_batches([len(p) for p in prompts], 8, 3, 192, 64, None, 3) == [[0, 1], [2, 3], [4, 5, 6]]
    first_steps = [ids for ids in engine.steps if all(len(engine.fed[i]) >= 1 for i in ids)]
    assert engine.steps[0] == [("gen", 0), ("gen", 1), ("gen", 2)]
    assert engine.peak_live == 3 and first_steps
    assert [i for i in engine.ended] == [("gen", i) for i in range(7)]


def test_request_numbers_and_steps_reach_the_chooser():
    seen = []

    def choose(logits, request_indices, steps):
        seen.append((list(request_indices), list(steps)))
        return [0] * len(request_indices)

    run_generation(ScriptedEngine(), [[1], [2, 3]], GenerationParams(max_new_tokens=3), choose, request_offset=100)
    assert seen == [([100, 101], [0, 0]), ([100, 101], [1, 1]), ([100, 101], [2, 2])]


def test_longest_sequence_ends_generation():
    engine = ScriptedEngine(max_seq_len=6)
    out = run_generation(engine, [[1, 2, 3, 4]], GenerationParams(max_new_tokens=10), chooser_from({0: list(range(50, 60))}))
    # positions 0..5 may be cached: the prompt and two fed tokens; the third chosen token is the last
    assert out == [[50, 51, 52]]
    assert engine.fed[("gen", 0)] == [1, 2, 3, 4, 50, 51]


def test_refusals_and_edge_cases():
    engine = ScriptedEngine(n_pages=2)
    with pytest.raises(ValueError, match="empty prompt"):
        run_generation(engine, [[1], []], GenerationParams(), chooser_from({}))
    with pytest.raises(ValueError, match="needs room"):
        run_generation(engine, [[1] * 200], GenerationParams(max_new_tokens=1), chooser_from({}))
    with pytest.raises(ValueError, match="exceeds the longest"):
        run_generation(ScriptedEngine(max_seq_len=3), [[1] * 4], GenerationParams(), chooser_from({}))
    assert run_generation(engine, [[1]], GenerationParams(max_new_tokens=0), chooser_from({})) == [[]]
    assert run_generation(engine, [], GenerationParams(), chooser_from({})) == []
    assert engine.steps == []


def test_storage_is_given_back_when_a_step_fails():
    engine = ScriptedEngine()

    def choose(logits, request_indices, steps):
        if steps[0] == 2:
            raise RuntimeError("boom")
        return [1] * len(request_indices)

    with pytest.raises(RuntimeError):
        run_generation(engine, [[1], [2]], GenerationParams(max_new_tokens=5), choose)
    assert engine.slot_of == {}


# ---------------------------------------------------------------------------------------------------------
# the loop that runs the device one step ahead of the host
class AheadEngine(ScriptedEngine):
    """Also takes a step's tokens "from the device" (here: a list the loop has not looked into)."""

    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.device_steps = []

    def decode_on_device(self, request_ids, tokens):
        assert len(request_ids) == len(tokens) and all(i in self.slot_of for i in request_ids)
        for i, t in zip(request_ids, tokens):
            self.fed[i].append(t)
        self.steps.append(list(request_ids))
        self.device_steps.append(list(request_ids))
        return [(i, list(self.fed[i])) for i in request_ids]


def ahead_chooser_from(plan, log):
    from gtar_kimik3_public_b200.engine.generation import DeviceChooser

    def choose(logits, request_indices, steps):
        return [plan[r][s] if s < len(plan[r]) else -1 for r, s in zip(request_indices, steps)]

    def fetch(tokens):
        log.append(("fetch", list(tokens)))
        return lambda: list(tokens)

    def take(tokens, rows):
        return [tokens[i] for i in rows]

    return DeviceChooser(choose, fetch, take)


@pytest.mark.parametrize("prompts,plan,max_new,stops", [
    ([[1, 2, 3], [4], [5, 6, 7, 8, 9]], {0: [10, 11, 99, 12], 1: [20, 21, 22, 23, 24], 2: [99]}, 4, {99}),
    ([[1], [2, 3]], {0: [5, 6, 7], 1: [99, 1, 1]}, 3, {99}),
    ([[1, 2]], {0: [7, 8, 9, 10, 11]}, 1, set()),
    ([[1] * 10, [2] * 70, [3] * 30, [4] * 64, [5] * 5], {i: [7, 8, 99, 9, 9, 9, 9, 9] for i in range(5)}, 8, {99}),
])
def test_loop_one_step_ahead_gives_the_same_tokens(prompts, plan, max_new, stops):
    params = GenerationParams(max_new_tokens=max_new, stop_ids=frozenset(stops), max_batch=3)
    plain_engine = ScriptedEngine(n_pages=6, max_seqs=3)
    want = run_generation(plain_engine, prompts, params, chooser_from(plan))
    log = []
    engine = AheadEngine(n_pages=6, max_seqs=3)
    got = run_generation(engine, prompts, params, chooser_from(plan), device_chooser=ahead_chooser_from(plan, log))
    assert got == want
    assert engine.slot_of == {} and sorted(map(str, engine.ended)) == sorted(map(str, plain_engine.ended))
    for request, fed in plain_engine.fed.items():
        # the same tokens were fed, except that a sequence that chose a stop token was fed it once more
        extra = engine.fed[request][len(fed):]
        assert engine.fed[request][:len(fed)] == fed and len(extra) <= 1
        if extra:
            assert extra[0] in stops
    # no step is launched for a sequence that has reached max_new_tokens
    for request, fed in engine.fed.items():
        assert len(fed) <= len(prompts[request[1]]) + max_new - 1


def test_loop_one_step_ahead_respects_the_longest_sequence():
    prompts = [[1] * 5, [2] * 3]
    plan = {0: [7] * 20, 1: [8] * 20}
    params = GenerationParams(max_new_tokens=20)
    want = run_generation(ScriptedEngine(max_seq_len=8), prompts, params, chooser_from(plan))
    engine = AheadEngine(max_seq_len=8)
    got = run_generation(engine, prompts, params, chooser_from(plan), device_chooser=ahead_chooser_from(plan, []))
    assert got == want and [len(o) for o in got] == [4, 6]
    assert max(len(f) for f in engine.fed.values()) <= 8

"""Generality of the layer parts: a toy mixer that keeps a state of its own (a decaying sum of
its inputs, one vector per sequence) is defined HERE, registered, put into a toy architecture
beside attention layers — with a run list that names a layer twice and lets an entry read
another entry's keys and values — written as a random model folder, loaded, and stepped through
the engine, without any change to the library's files.  It is a test fixture, not a model of
anyone's."""

import dataclasses
from typing import ClassVar

import pytest
import torch

from tests.plain import model as plain
from tests.plain.weights import read_safetensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def define_toy():
    from gtar_kimik3_public_b200.config.base import ModelConfig
    from gtar_kimik3_public_b200.models.model import ModelPlan, RunEntry
    from gtar_kimik3_public_b200.ops.linear import linear
    from gtar_kimik3_public_b200.parts.base import Mixer, StateRequest, TensorSpec, build_part, register_part
    from gtar_kimik3_public_b200.parts.embedding import OutputHead, TokenEmbedding
    from gtar_kimik3_public_b200.registry import register_architecture

    class DecayingSumMixer(Mixer):
        """state <- sigmoid(gate) * state + x_t ;  out_t = state @ W.T   (state: [hidden], float32)."""

        def __init__(self, hidden_size):
            self.hidden_size = hidden_size

        def tensor_specs(self):
            return {"gate": TensorSpec((self.hidden_size,), "vector"), "proj.weight": TensorSpec((self.hidden_size,) * 2)}

        def load(self, tensors):
            self.gate, self.proj = tensors["gate"].float(), tensors["proj.weight"].contiguous()

        def cache_request(self):
            return StateRequest((self.hidden_size,), torch.float32)

        def forward(self, x, ctx, state):
            decay = torch.sigmoid(self.gate)
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            start = 0
            for slot, n in zip(ctx.host_slots, ctx.host_q_len):
                s = state[slot]
                for t in range(start, start + n):
                    s = decay * s + x[t].float()
                    out[t] = s
                state[slot] = s
                start += n
            return linear(out.to(x.dtype), self.proj)

    class TwoStateMixer(Mixer):
        """A mixer with TWO states of their own shapes, made of device-side operations only, so that its steps
        may be captured in CUDA graphs (``graph_safe``):

            sum   <- sigmoid(gate) * sum + x_t            (state 0: [hidden], float32)
            out_t  = (sum + 0.5 * x_{t-1} + 0.25 * x_{t-2}) @ W.T
            last  <- (x_t, x_{t-1})                        (state 1: [2, hidden], float32, a rolling buffer)

        Every per-step number (slots, starts of the sequences' tokens) is read from device memory; the only host
        number is the longest part of the step, which belongs to a captured step's shape."""

        graph_safe = True

        def __init__(self, hidden_size):
            self.hidden_size = hidden_size

        def tensor_specs(self):
            return {"gate": TensorSpec((self.hidden_size,), "vector"), "proj.weight": TensorSpec((self.hidden_size,) * 2)}

        def load(self, tensors):
            self.gate, self.proj = tensors["gate"].float(), tensors["proj.weight"].contiguous()

        def cache_request(self):
            return [StateRequest((self.hidden_size,), torch.float32), StateRequest((2, self.hidden_size), torch.float32)]

        def forward(self, x, ctx, states):
            total, last = states
            decay = torch.sigmoid(self.gate)
            slots = ctx.slots.long()
            starts, counts = ctx.cu_q[:-1].long(), (ctx.cu_q[1:] - ctx.cu_q[:-1]).long()
            s, prev = total[slots], last[slots]  # [n_seqs, hidden], [n_seqs, 2, hidden]
            out = torch.zeros((ctx.n_tokens + 1, self.hidden_size), dtype=torch.float32, device=x.device)
            xf = x.float()
            for j in range(ctx.max_q_len):
                valid = (counts > j)[:, None]
                rows = torch.where(counts > j, starts + j, torch.full_like(starts, ctx.n_tokens))  # the spare row takes the rest
                x_j = xf[(starts + j).clamp(max=ctx.n_tokens - 1)]
                s = torch.where(valid, decay * s + x_j, s)
                out[rows] = s + 0.5 * prev[:, 0] + 0.25 * prev[:, 1]
                prev = torch.where(valid[:, :, None], torch.stack([x_j, prev[:, 0]], dim=1), prev)
            total[slots] = s
            last[slots] = prev
            return linear(out[:-1].to(x.dtype), self.proj)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab_size: int
        hidden_size: int
        intermediate_size: int
        num_attention_heads: int
        num_key_value_heads: int
        head_dim: int
        rms_norm_eps: float
        rope_theta: float
        run_list: list
        middle_mixer: str = "toy_decaying_sum"
        initializer_range: float | None = None
        max_position_embeddings: int | None = None
        ARCH_NAMES: ClassVar[tuple] = ("toy_state_arch",)

    def build_plan(c):
        rope = build_part("position", "rope", dim=c.head_dim, base=c.rope_theta)

        def layer(mixer):
            return build_part(
                "block", "pre_norm", input_norm=build_part("norm", "rmsnorm", size=c.hidden_size, eps=c.rms_norm_eps),
                mixer=mixer, post_norm=build_part("norm", "rmsnorm", size=c.hidden_size, eps=c.rms_norm_eps),
                feed_forward=build_part("feed_forward", "swiglu", hidden_size=c.hidden_size, intermediate_size=c.intermediate_size))

        def attention():
            return build_part("mixer", "gqa_attention", hidden_size=c.hidden_size, n_q_heads=c.num_attention_heads,
                              n_kv_heads=c.num_key_value_heads, head_dim=c.head_dim, qk_norm_eps=c.rms_norm_eps, position=rope)

        layers = [layer(attention()), layer(build_part("mixer", c.middle_mixer, hidden_size=c.hidden_size)), layer(attention())]
        emb = TokenEmbedding(c.vocab_size, c.hidden_size)
        return ModelPlan(embedding=emb, layers=layers, final_norm=build_part("norm", "rmsnorm", size=c.hidden_size, eps=c.rms_norm_eps),
                         head=OutputHead(c.hidden_size, c.vocab_size, tied_to=emb),
                         run_list=[RunEntry(l, s) for l, s in c.run_list], positions=[rope])

    register_part("mixer", "toy_decaying_sum", DecayingSumMixer, replace=True)
    register_part("mixer", "toy_two_states", TwoStateMixer, replace=True)
    register_architecture(ToyConfig.ARCH_NAMES, ToyConfig, build_plan, replace=True)
    return ToyConfig


BASE = dict(arch="toy_state_arch", vocab_size=200, hidden_size=48, intermediate_size=80, num_attention_heads=3,
            num_key_value_heads=1, head_dim=16, rms_norm_eps=1e-5, rope_theta=1e4, initializer_range=0.1,
            max_position_embeddings=128)


def plain_toy_forward(ids, w, cfg, rolling=False):
    """Whole-sequence forward of the toy architecture with run list attention, toy, toy; ``rolling`` adds the
    second state's terms (half of the input before, a quarter of the one before that)."""
    eps = cfg["rms_norm_eps"]
    h = plain.embed(ids, w["model.embed_tokens.weight"])
    for layer in (0, 1, 1):
        p = f"model.layers.{layer}."
        x = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        if layer == 0:
            h = h + plain.attention_mixer(x, w, p + "self_attn.", cfg)
        else:
            decay = torch.sigmoid(w[p + "self_attn.gate"])
            s, rows = torch.zeros_like(x[0]), []
            for t in range(x.shape[0]):
                s = decay * s + x[t]
                extra = 0
                if rolling:
                    extra = (0.5 * x[t - 1] if t >= 1 else 0) + (0.25 * x[t - 2] if t >= 2 else 0)
                rows.append(s + extra)
            h = h + torch.stack(rows) @ w[p + "self_attn.proj.weight"].T
        h = h + plain.swiglu(plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return plain.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T


@pytest.mark.parametrize("run_list,compare_plain", [([[0, None], [1, None], [1, None]], True),
                                                     ([[0, None], [1, None], [2, 0], [1, None]], False)])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, run_list, compare_plain):
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    define_toy()
    cfg = {**BASE, "run_list": run_list}
    config = config_from_dict(cfg)
    folder = write_random_model(tmp_path, config, seed=4)
    model = load(folder, "float32")
    layout = model.cache_layout()
    assert [type(r).__name__ for r in layout.requests][:2] == ["KVRequest", "StateRequest"]
    engine = Engine(model, max_tokens=512, max_seqs=3)
    assert len(engine.cache.state_groups) == 1
    assert engine.cache.state_groups[0].state.shape[0] == sum(1 for l, _ in run_list if l == 1)  # a state per run, not per layer
    gen = torch.Generator().manual_seed(0)
    requests = [torch.randint(0, 200, (n,), generator=gen).tolist() for n in (40, 7, 90)]
    whole = []
    for r, tokens in enumerate(requests):
        whole.append(engine.step([StepEntry(("w", r), tokens, list(range(len(tokens))))]))
        engine.end([("w", r)])
    if compare_plain:
        w = {k: v.double() for k, v in read_safetensors(folder / "model.safetensors").items()}
        for tokens, got in zip(requests, whole):
            want = plain_toy_forward(torch.tensor(tokens), w, cfg)
            assert (got.double().cpu() - want).abs().max() < 1e-4
    # the same requests as one batch of unequal lengths: prompts of 5 tokens, then one token each;
    # slots are used again (the whole runs above held them), so a state that is not zeroed would show
    fed = {r: 5 for r in range(3)}
    rows = {r: [] for r in range(3)}
    logits = engine.step([StepEntry(r, requests[r][:5], list(range(5))) for r in range(3)])
    for r in range(3):
        rows[r].append(logits[5 * r:5 * r + 5])
    live = [0, 1, 2]
    while live:
        logits = engine.step([StepEntry(r, [requests[r][fed[r]]], [0]) for r in live])
        for i, r in enumerate(live):
            rows[r].append(logits[i:i + 1])
            fed[r] += 1
        done = [r for r in live if fed[r] == len(requests[r])]
        engine.end(done)
        live = [r for r in live if r not in done]
    for r in range(3):
        assert (torch.cat(rows[r]) - whole[r]).abs().max() < 2e-5, f"request {r}: cutting changed the logits"
    assert engine.cache.slots.n_used == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_safe_mixer_with_two_states_steps_once_per_step(tmp_path, dtype):
    """A kernel-only mixer that advances two states in place, run from CUDA graphs: whole, token by token and in a
    batch of unequal lengths give the same logits, so no step (not even the one at which a shape is captured)
    advanced a state twice, and both states follow their slot."""
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    define_toy()
    cfg = {**BASE, "run_list": [[0, None], [1, None], [1, None]], "middle_mixer": "toy_two_states"}
    folder = write_random_model(tmp_path, config_from_dict(cfg), seed=6)
    model = load(folder, dtype)
    assert model.graph_safe()
    layout = model.cache_layout()
    assert [type(r).__name__ for r in layout.requests[1]] == ["StateRequest", "StateRequest"]
    engine = Engine(model, max_tokens=512, max_seqs=3)
    assert engine.graphs is not None
    assert sorted(tuple(g.state.shape) for g in engine.cache.state_groups) == [(2, 3, 2, 48), (2, 3, 48)]
    gen = torch.Generator().manual_seed(1)
    requests = [torch.randint(0, 200, (n,), generator=gen).tolist() for n in (30, 6, 55)]
    w = {k: v.double() for k, v in read_safetensors(folder / "model.safetensors").items()}
    want = [plain_toy_forward(torch.tensor(tokens), w, cfg, rolling=True) for tokens in requests]
    tolerance = 1e-4 if dtype == "float32" else 0.08

    def close(got, r, what):
        err = (got.double().cpu() - want[r]).abs().max().item()
        assert err < tolerance, f"{what}, request {r}: differs from the plain forward by {err:.3e}"

    for repeat in range(3):  # whole prompts: a shape's first, second (captured) and third (replayed) appearance
        for r, tokens in enumerate(requests):
            close(engine.step([StepEntry(("w", r), tokens, list(range(len(tokens))))]), r, f"whole, time {repeat}")
            engine.end([("w", r)])
    for r, tokens in enumerate(requests):  # token by token: every step a decode step (captured at its first use)
        rows = [engine.step([StepEntry(("t", r), [token], [0])]) for token in tokens]
        engine.end([("t", r)])
        close(torch.cat(rows), r, "token by token")
    fed = {r: 4 for r in range(3)}  # a batch of unequal lengths whose shorter requests end earlier
    rows = {r: [] for r in range(3)}
    logits = engine.step([StepEntry(r, requests[r][:4], list(range(4))) for r in range(3)])
    for r in range(3):
        rows[r].append(logits[4 * r:4 * r + 4])
    live = [0, 1, 2]
    while live:
        logits = engine.step([StepEntry(r, [requests[r][fed[r]]], [0]) for r in live])
        for i, r in enumerate(live):
            rows[r].append(logits[i:i + 1])
            fed[r] += 1
        done = [r for r in live if fed[r] == len(requests[r])]
        engine.end(done)
        live = [r for r in live if r not in done]
    for r in range(3):
        close(torch.cat(rows[r]), r, "batched")
    assert len(engine.graphs.graphs) >= 3
    assert engine.cache.slots.n_used == 0

"""Generality of the layer parts, second sheet: a feed-forward with routing (top-1 of a few experts),
another position encoding (only some pairs of a head rotate, with angles linear in the pair's index)
and another norm (mean-free scaling) are defined HERE, registered, mixed layer by layer with the
library's own parts in a toy architecture, written as a random model folder, loaded and stepped
through the engine without any change to the library's files.  The host work the toy parts do keeps
the model out of CUDA graphs by itself (they do not declare ``graph_safe``).  Test fixtures, not
models of anyone's."""

import dataclasses
from typing import ClassVar

import pytest
import torch

from tests.plain import model as plain
from tests.plain.weights import read_safetensors

pytestmark = pytest.mark.gpu
N_EXPERTS = 3
ROTATING_PAIRS = 5
ANGLE_STEP = 0.07


def toy_tables(positions: torch.Tensor, head_dim: int):
    """cos, sin [T, head_dim / 2]: pair j < ROTATING_PAIRS turns by pos * (j + 1) * ANGLE_STEP, the rest not at all."""
    half = head_dim // 2
    rate = torch.zeros(half, dtype=torch.float32)
    rate[:ROTATING_PAIRS] = (torch.arange(ROTATING_PAIRS, dtype=torch.float32) + 1) * ANGLE_STEP
    angles = positions.to(torch.float32)[:, None] * rate[None, :]
    return angles.cos(), angles.sin()


def define_toy():
    from gtar_kimik3_public_b200.config.base import ModelConfig
    from gtar_kimik3_public_b200.models.model import ModelPlan, RunEntry
    from gtar_kimik3_public_b200.ops.linear import linear
    from gtar_kimik3_public_b200.parts.base import FeedForward, Norm, PositionEncoding, TensorSpec, build_part, register_part
    from gtar_kimik3_public_b200.parts.embedding import OutputHead, TokenEmbedding
    from gtar_kimik3_public_b200.registry import register_architecture

    class Top1Experts(FeedForward):
        """out_t = p_t[e] * down_e(silu(up_e(x_t))),  p_t = softmax(x_t R^T) in 32-bit,  e = argmax p_t."""

        def __init__(self, hidden_size, intermediate_size, n_experts):
            self.hidden_size, self.intermediate_size, self.n_experts = hidden_size, intermediate_size, n_experts

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec((self.n_experts, self.hidden_size))}
            for e in range(self.n_experts):
                specs[f"experts.{e}.up.weight"] = TensorSpec((self.intermediate_size, self.hidden_size))
                specs[f"experts.{e}.down.weight"] = TensorSpec((self.hidden_size, self.intermediate_size))
            return specs

        def load(self, tensors):
            self.router = tensors["router.weight"].float()
            self.up = [tensors[f"experts.{e}.up.weight"].contiguous() for e in range(self.n_experts)]
            self.down = [tensors[f"experts.{e}.down.weight"].contiguous() for e in range(self.n_experts)]

        def forward(self, x, ctx):
            probs = torch.softmax(x.float() @ self.router.T, dim=-1)
            weight, expert = probs.max(dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.n_experts):
                rows = (expert == e).nonzero().flatten()  # waits for the device: this part is not graph-safe
                if rows.numel():
                    hidden = torch.nn.functional.silu(linear(x[rows].contiguous(), self.up[e]).float()).to(x.dtype)
                    out[rows] = linear(hidden, self.down[e]).float() * weight[rows, None]
            return out.to(x.dtype)

    class PartialLinearRotation(PositionEncoding):
        def __init__(self, dim):
            self.dim, self.cos, self.sin = dim, None, None

        def prepare(self, max_position, device):
            if self.cos is None or self.cos.shape[0] <= max_position or self.cos.device != device:
                cos, sin = toy_tables(torch.arange(max(max_position + 1, 64)), self.dim)
                self.cos, self.sin = cos.to(device).contiguous(), sin.to(device).contiguous()

    class MeanFreeScale(Norm):
        """y = weight * (v - mean(v)),  v = h + delta (added into the stream unless only some rows are asked for)."""

        def __init__(self, size):
            self.size = size

        def tensor_specs(self):
            return {"weight": TensorSpec((self.size,), "vector")}

        def load(self, tensors):
            self.weight = tensors["weight"].float()

        def forward(self, h, delta, out_dtype, rows=None):
            if rows is not None:
                v = h[rows.long()] if delta is None else h[rows.long()] + delta[rows.long()].float()
            else:
                if delta is not None:
                    h += delta.float()
                v = h
            return (self.weight * (v - v.mean(dim=-1, keepdim=True))).to(out_dtype)

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
        initializer_range: float | None = None
        max_position_embeddings: int | None = None
        ARCH_NAMES: ClassVar[tuple] = ("toy_parts_arch",)

    def build_plan(c):
        toy_position = build_part("position", "toy_partial_linear", dim=c.head_dim)
        rope = build_part("position", "rope", dim=c.head_dim, base=c.rope_theta)

        def rmsnorm():
            return build_part("norm", "rmsnorm", size=c.hidden_size, eps=c.rms_norm_eps)

        def attention(position):
            return build_part("mixer", "gqa_attention", hidden_size=c.hidden_size, n_q_heads=c.num_attention_heads,
                              n_kv_heads=c.num_key_value_heads, head_dim=c.head_dim, qk_norm_eps=c.rms_norm_eps, position=position)

        layers = [
            # layer 0: toy norm in front of attention with the toy rotation, then the routed feed-forward
            build_part("block", "pre_norm", input_norm=build_part("norm", "toy_mean_free", size=c.hidden_size),
                       mixer=attention(toy_position), post_norm=rmsnorm(),
                       feed_forward=build_part("feed_forward", "toy_top1_experts", hidden_size=c.hidden_size,
                                               intermediate_size=c.intermediate_size, n_experts=N_EXPERTS)),
            # layer 1: the library's own parts
            build_part("block", "pre_norm", input_norm=rmsnorm(), mixer=attention(rope), post_norm=rmsnorm(),
                       feed_forward=build_part("feed_forward", "swiglu", hidden_size=c.hidden_size,
                                               intermediate_size=c.intermediate_size)),
        ]
        emb = TokenEmbedding(c.vocab_size, c.hidden_size)
        return ModelPlan(embedding=emb, layers=layers, final_norm=rmsnorm(), head=OutputHead(c.hidden_size, c.vocab_size, tied_to=emb),
                         run_list=[RunEntry(0, None), RunEntry(1, None)], positions=[toy_position, rope])

    register_part("feed_forward", "toy_top1_experts", Top1Experts, replace=True)
    register_part("position", "toy_partial_linear", PartialLinearRotation, replace=True)
    register_part("norm", "toy_mean_free", MeanFreeScale, replace=True)
    register_architecture(ToyConfig.ARCH_NAMES, ToyConfig, build_plan, replace=True)


CFG = dict(arch="toy_parts_arch", vocab_size=180, hidden_size=40, intermediate_size=56, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5, rope_theta=1e4, initializer_range=0.15,
           max_position_embeddings=128)


def plain_attention(x, w, prefix, cfg, cos, sin):
    """tests/plain/model.py's attention_mixer with the rotation tables given ([T, d/2], repeated to [T, d])."""
    n_q, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    t = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(t, n_q, d)
    k = (x @ w[prefix + "k_proj.weight"].T).view(t, n_kv, d)
    v = (x @ w[prefix + "v_proj.weight"].T).view(t, n_kv, d)
    q = plain.rms_norm(q, w[prefix + "q_norm.weight"], cfg["rms_norm_eps"])
    k = plain.rms_norm(k, w[prefix + "k_norm.weight"], cfg["rms_norm_eps"])
    cos, sin = torch.cat((cos, cos), dim=-1), torch.cat((sin, sin), dim=-1)
    o = plain.causal_gqa_attention(plain.apply_rotary(q, cos, sin), plain.apply_rotary(k, cos, sin), v)
    return o.reshape(t, n_q * d) @ w[prefix + "o_proj.weight"].T


def plain_toy_forward(ids, w, cfg):
    eps, t = cfg["rms_norm_eps"], ids.shape[0]
    h = plain.embed(ids, w["model.embed_tokens.weight"])
    # layer 0
    p = "model.layers.0."
    x = w[p + "input_layernorm.weight"] * (h - h.mean(dim=-1, keepdim=True))
    cos, sin = toy_tables(torch.arange(t), cfg["head_dim"])
    h = h + plain_attention(x, w, p + "self_attn.", cfg, cos.double(), sin.double())
    x = plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    probs = torch.softmax(x @ w[p + "mlp.router.weight"].T, dim=-1)
    weight, expert = probs.max(dim=-1)
    branch = torch.zeros_like(h)
    for i in range(t):
        e = int(expert[i])
        hidden = torch.nn.functional.silu(x[i] @ w[p + f"mlp.experts.{e}.up.weight"].T)
        branch[i] = weight[i] * (hidden @ w[p + f"mlp.experts.{e}.down.weight"].T)
    h = h + branch
    # layer 1
    p = "model.layers.1."
    x = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps)
    h = h + plain.attention_mixer(x, w, p + "self_attn.", cfg)
    h = h + plain.swiglu(plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return plain.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T


def test_toy_feed_forward_position_and_norm_are_registered_built_and_stepped(tmp_path):
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    define_toy()
    config = config_from_dict(CFG)
    folder = write_random_model(tmp_path, config, seed=11)
    names = set(read_safetensors(folder / "model.safetensors"))
    assert "model.layers.0.mlp.router.weight" in names and "model.layers.0.mlp.experts.2.down.weight" in names
    assert "model.layers.1.mlp.gate_proj.weight" in names and "model.layers.0.mlp.gate_proj.weight" not in names
    model = load(folder, "float32")
    assert not model.graph_safe()  # the toy parts do host work; the library's own layer alone would be safe
    assert model.plan.layers[1].graph_safe and not model.plan.layers[0].graph_safe
    engine = Engine(model, max_tokens=512, max_seqs=3)
    assert engine.graphs is None
    gen = torch.Generator().manual_seed(3)
    requests = [torch.randint(0, CFG["vocab_size"], (n,), generator=gen).tolist() for n in (50, 9, 77)]
    w = {k: v.double() for k, v in read_safetensors(folder / "model.safetensors").items()}
    whole = []
    for r, tokens in enumerate(requests):
        got = engine.step([StepEntry(("w", r), tokens, list(range(len(tokens))))])
        engine.end([("w", r)])
        want = plain_toy_forward(torch.tensor(tokens), w, CFG)
        assert (got.double().cpu() - want).abs().max() < 1e-4, f"request {r} differs from the plain toy forward"
        whole.append(got)
    # unequal batch: prompts of 4 tokens, then one token each, shorter requests ending earlier
    fed, rows = {r: 4 for r in range(3)}, {r: [] for r in range(3)}
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
        assert (torch.cat(rows[r]) - whole[r]).abs().max() < 2e-5, f"request {r}: cutting changed the logits"
    assert engine.cache.slots.n_used == 0


def test_toy_parts_run_in_bfloat16_too(tmp_path):
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    define_toy()
    folder = write_random_model(tmp_path, config_from_dict(CFG), seed=11)
    tokens = torch.randint(0, CFG["vocab_size"], (33,), generator=torch.Generator().manual_seed(5)).tolist()
    outs = {}
    for dtype in ("float32", "bfloat16"):
        engine = Engine(load(folder, dtype), max_tokens=128, max_seqs=1)
        outs[dtype] = engine.step([StepEntry(0, tokens, list(range(len(tokens))))]).float().cpu()
        engine.end([0])
    # a token near a routing tie may go to another expert in bfloat16: look at the bulk, not the worst place
    err = (outs["bfloat16"] - outs["float32"]).abs().amax(dim=-1)
    assert err.median() < 0.05 * outs["float32"].abs().max()

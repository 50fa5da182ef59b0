"""Each part of a layer alone — norm, position encoding, attention mixer, feed-forward, block,
embedding and head — built from numbers (sizes other than the tiny models') and compared with
the plain function of the same part on a whole sequence."""

import pytest
import torch

from tests.plain import model as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


def lowp(function, *args):
    """The plain function with every matrix product rounded to bfloat16, in float32: the standard low-precision
    implementation that the bfloat16 results are measured against."""
    def narrow(value):
        if torch.is_tensor(value):
            return value.float()
        if isinstance(value, dict):
            return {k: narrow(v) for k, v in value.items()}
        return value

    plain.LOWP = torch.bfloat16
    try:
        return function(*[narrow(a) for a in args]).double()
    finally:
        plain.LOWP = None


def assert_close(got, want, dtype, yard_result=None, what=""):
    """float32: within 1e-4 of the float64 result.  bfloat16: at most twice the error of the standard low-precision
    implementation plus 1e-4 (the reference's rule, tests/test_flash_attention_2.py:54-58); where the part has no
    matrix product (a norm), within one bfloat16 rounding of each value."""
    got = got.double().cpu()
    err = (got - want).abs().max().item()
    if dtype == torch.float32:
        assert err < 1e-4, f"{what}: float32 differs by {err:.3e}"
    elif yard_result is None:
        assert ((got - want).abs() <= want.abs() * 2.0**-8 + 1e-6).all(), f"{what}: more than one bfloat16 rounding off ({err:.3e})"
    else:
        yard = (yard_result - want).abs().max().item()
        assert err <= 2 * yard + 1e-4, f"{what}: bfloat16 error {err:.3e} exceeds twice the yardstick {yard:.3e}"


def load_part(part, tensors, dtype):
    """Hands a part its tensors the way the loader does: matrices in the run dtype, vectors 32-bit."""
    specs = part.tensor_specs()
    out = {}
    for name, t in tensors.items():
        keep = torch.float32 if (dtype == torch.float32 or specs[name].kind == "vector") else torch.bfloat16
        out[name] = t.to(keep).to(DEV)
    part.load(out)


def one_sequence_ctx(n, dtype, n_kv, d, want=None):
    """A cache and a step context for one whole sequence of n tokens."""
    from gtar_kimik3_public_b200.cache import Cache, CacheLayout
    from gtar_kimik3_public_b200.engine.step import SequenceStep, plan_step
    from gtar_kimik3_public_b200.parts.base import KVRequest

    cache = Cache(CacheLayout([KVRequest(n_kv, d)]), max_tokens=n + 64, dtype=dtype, device=DEV)
    slot = cache.open()
    cache.grow(slot, n)
    cache.sync()
    ctx = plan_step([SequenceStep(slot, 0, [0] * n, want or [])], dtype, torch.device(DEV), 1)
    return cache, ctx


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from gtar_kimik3_public_b200.parts import build_part

    norm = build_part("norm", "rmsnorm", size=200, eps=1e-5)
    w = 1 + 0.1 * rand(200, seed=1)
    load_part(norm, {"weight": w}, dtype)
    h = rand(9, 200, seed=2).float()
    delta = rand(9, 200, seed=3).to(dtype)
    hd = h.to(DEV)
    out = norm.forward(hd, delta.to(DEV), dtype)
    want = plain.rms_norm(h.double() + delta.double(), w.float().double(), 1e-5)
    assert out.dtype == dtype
    assert_close(out, want, dtype, None, "rmsnorm")


def test_rotary_tables_match_the_reference_expression():
    from gtar_kimik3_public_b200.parts import build_part

    for dim, base in ((16, 1e4), (48, 1e6), (128, 5e5)):
        rope = build_part("position", "rope", dim=dim, base=base)
        rope.prepare(4095, torch.device(DEV))
        cos, sin = plain.rotary_tables(torch.arange(4096), dim, base)
        assert rope.cos.shape == (4096, dim // 2)
        # same float32 angle; the device's cos/sin may differ from the host's in the last place
        assert (rope.cos.cpu() - cos[:, : dim // 2]).abs().max() < 5e-7
        assert (rope.sin.cpu() - sin[:, : dim // 2]).abs().max() < 5e-7
        rope.prepare(10, torch.device(DEV))
        assert rope.cos.shape[0] == 4096  # not shrunk, not rebuilt


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,n_q,n_kv,d", [(96, 6, 2, 48), (72, 4, 4, 16)])
def test_attention_mixer(dtype, hidden, n_q, n_kv, d):
    from gtar_kimik3_public_b200.parts import build_part

    eps, theta, n = 1e-5, 1e5, 150
    rope = build_part("position", "rope", dim=d, base=theta)
    mixer = build_part("mixer", "gqa_attention", hidden_size=hidden, n_q_heads=n_q, n_kv_heads=n_kv, head_dim=d,
                       qk_norm_eps=eps, position=rope)
    w = {
        "q_proj.weight": rand(n_q * d, hidden, seed=1, scale=0.1), "k_proj.weight": rand(n_kv * d, hidden, seed=2, scale=0.1),
        "v_proj.weight": rand(n_kv * d, hidden, seed=3, scale=0.1), "o_proj.weight": rand(hidden, n_q * d, seed=4, scale=0.1),
        "q_norm.weight": 1 + 0.1 * rand(d, seed=5), "k_norm.weight": 1 + 0.1 * rand(d, seed=6),
    }
    w = {k: v.to(torch.bfloat16).double() if "proj" in k else v.float().double() for k, v in w.items()}
    load_part(mixer, w, dtype)
    x = rand(n, hidden, seed=7).to(dtype)
    cache, ctx = one_sequence_ctx(n, dtype, n_kv, d)
    rope.prepare(n, torch.device(DEV))
    out = mixer.forward(x.to(DEV), ctx, cache.view(0))
    cfg = {"num_attention_heads": n_q, "num_key_value_heads": n_kv, "head_dim": d, "rms_norm_eps": eps, "rope_theta": theta}
    want = plain.attention_mixer(x.double(), w, "", cfg)
    assert_close(out, want, dtype, lowp(plain.attention_mixer, x, w, "", cfg), "attention mixer")


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_feed_forward(dtype):
    from gtar_kimik3_public_b200.parts import build_part

    ffn = build_part("feed_forward", "swiglu", hidden_size=72, intermediate_size=200)
    w = {"gate_proj.weight": rand(200, 72, seed=1, scale=0.2), "up_proj.weight": rand(200, 72, seed=2, scale=0.2),
         "down_proj.weight": rand(72, 200, seed=3, scale=0.2)}
    w = {k: v.to(torch.bfloat16).double() for k, v in w.items()}
    load_part(ffn, w, dtype)
    x = rand(11, 72, seed=4).to(dtype)
    out = ffn.forward(x.to(DEV), None)
    want = plain.swiglu(x.double(), w, "")
    assert_close(out, want, dtype, lowp(plain.swiglu, x, w, ""), "feed-forward")


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block_and_pending_add(dtype):
    from gtar_kimik3_public_b200.parts import build_part

    hidden, n_q, n_kv, d, inter, eps, theta, n = 80, 4, 2, 32, 144, 1e-6, 1e4, 70
    rope = build_part("position", "rope", dim=d, base=theta)
    block = build_part(
        "block", "pre_norm", input_norm=build_part("norm", "rmsnorm", size=hidden, eps=eps),
        mixer=build_part("mixer", "gqa_attention", hidden_size=hidden, n_q_heads=n_q, n_kv_heads=n_kv, head_dim=d,
                         qk_norm_eps=eps, position=rope),
        post_norm=build_part("norm", "rmsnorm", size=hidden, eps=eps),
        feed_forward=build_part("feed_forward", "swiglu", hidden_size=hidden, intermediate_size=inter))
    specs = block.tensor_specs()
    assert len(specs) == 11
    w = {}
    for i, (name, spec) in enumerate(specs.items()):
        if spec.kind == "vector":
            w[name] = (1 + 0.1 * rand(*spec.shape, seed=i)).float().double()
        else:
            w[name] = rand(*spec.shape, seed=i, scale=0.1).to(torch.bfloat16).double()
    load_part(block, w, dtype)
    h = rand(n, hidden, seed=50).float()
    cache, ctx = one_sequence_ctx(n, dtype, n_kv, d)
    rope.prepare(n, torch.device(DEV))
    hd = h.to(DEV)
    stream, pending = block.forward(hd, None, ctx, cache.view(0))
    got = stream.double().cpu() + pending.double().cpu()  # the stream after the layer = stream + pending
    cfg = {"num_attention_heads": n_q, "num_key_value_heads": n_kv, "head_dim": d, "rms_norm_eps": eps, "rope_theta": theta}
    named = {"model.layers.0." + k: v for k, v in w.items()}
    want = plain.block(h.double(), named, 0, cfg)
    assert_close(got, want, dtype, lowp(plain.block, h, named, 0, cfg), "block")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head(dtype, tied):
    from gtar_kimik3_public_b200.parts.embedding import OutputHead, TokenEmbedding

    vocab, hidden = 1000 + 7, 72
    emb = TokenEmbedding(vocab, hidden)
    head = OutputHead(hidden, vocab, tied_to=emb if tied else None)
    table = rand(vocab, hidden, seed=1, scale=0.1).to(torch.bfloat16).double()
    own = rand(vocab, hidden, seed=2, scale=0.1).to(torch.bfloat16).double()
    load_part(emb, {"weight": table}, dtype)
    load_part(head, {} if tied else {"weight": own}, dtype)
    ids = torch.tensor([0, 1006, 5], dtype=torch.int32)
    assert torch.equal(emb.forward(ids.to(DEV)).cpu().double(), table[ids.long()])
    z = rand(4, hidden, seed=3).to(dtype)
    logits = head.forward(z.to(DEV))
    want = z.double() @ (table if tied else own).T
    assert logits.dtype == torch.float32 and logits.shape == (4, vocab)
    assert_close(logits, want, dtype, lowp(plain.mm, z, (table if tied else own).T), "head")

"""Each kernel alone against a plain float64 formula, at sizes other than the tiny models':
widths and vocabularies that are no power of two, head sizes 16/48/80/128, groups of 1/2/3/4,
lengths 1/777/1000.  Where random inputs would hide a fault the inputs are made to show it: one
far key whose score stands out, a key at the window's edge, pages handed out in scrambled order
with every unused place poisoned."""

import math

import numpy as np
import pytest
import torch

from tests.plain import model as plain
from tests.plain import sampling as plain_sampling

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
BF16_ULP = 2.0**-8  # one unit in the last place of bfloat16, relative


def F():
    from gtar_kimik3_public_b200.ops import functional

    return functional


def rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


def close(got, want, dtype, what, atol=1e-5):
    got, want = got.double().cpu(), want.double()
    assert torch.isfinite(got).all(), what
    if dtype == torch.float32:
        err = ((got - want).abs() / (want.abs() + 1)).max().item()
        assert err < atol, f"{what}: {err:.3e}"
    else:  # a bfloat16 result is the rounded 32-bit value: within one unit in the last place
        err = ((got - want).abs() / (want.abs() + 1e-2)).max().item()
        assert err < 1.01 * BF16_ULP, f"{what}: {err:.3e}"


# ------------------------------------------------------------------ token-wise kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab,hidden", [(37, 80), (1000, 1536)])
def test_embed_rows(dtype, vocab, hidden):
    table = rand(vocab, hidden).to(dtype)
    ids = torch.tensor([0, vocab - 1, 5, 5, vocab // 2], dtype=torch.int32)
    out = F().embed_rows(table.to(DEV), ids.to(DEV))
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table.float()[ids.long()])


@pytest.mark.parametrize("hidden", [80, 1000, 5120])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("weight_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(hidden, out_dtype, weight_dtype):
    n, eps = 7, 3e-5
    h = rand(n, hidden, seed=1, scale=3.0).float()
    delta = rand(n, hidden, seed=2).to(out_dtype)
    w = (1 + 0.1 * rand(hidden, seed=3)).to(weight_dtype)
    want_h = h.double() + delta.double()
    want = plain.rms_norm(want_h, w.double(), eps)
    hd = h.to(DEV)
    got = F().add_rmsnorm(hd, delta.to(DEV), w.to(DEV), eps, out_dtype)
    close(got, want, out_dtype, "add_rmsnorm out")
    assert torch.equal(hd.cpu(), (h + delta.float()))  # the stream holds the 32-bit sum
    # without delta the stream is left alone
    hd2 = h.to(DEV)
    got2 = F().add_rmsnorm(hd2, None, w.to(DEV), eps, out_dtype)
    close(got2, plain.rms_norm(h.double(), w.double(), eps), out_dtype, "rmsnorm without delta")
    assert torch.equal(hd2.cpu(), h)
    # chosen rows: same numbers as the full call, stream untouched
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    hd3 = h.to(DEV)
    got3 = F().add_rmsnorm(hd3, delta.to(DEV), w.to(DEV), eps, out_dtype, rows=rows.to(DEV))
    assert torch.equal(got3.cpu(), got.cpu()[rows.long()]) and torch.equal(hd3.cpu(), h)


@pytest.mark.parametrize("hidden", [1024, 72, 900])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm_of_many_rows_equals_the_same_rows_a_few_at_a_time(hidden, out_dtype):
    """Many short rows take a kernel with a warp a row; its numbers are bit for bit those of the block-a-row kernel,
    so a row's norm does not depend on how many rows its step has."""
    n, eps = 515, 2e-6  # a last block with three rows
    h = rand(n, hidden, seed=11, scale=3.0).float()
    delta = rand(n, hidden, seed=12).to(out_dtype)
    w = (1 + 0.1 * rand(hidden, seed=13)).to(out_dtype)
    whole_h = h.to(DEV)
    whole = F().add_rmsnorm(whole_h, delta.to(DEV), w.to(DEV), eps, out_dtype)
    close(whole, plain.rms_norm(h.double() + delta.double(), w.double(), eps), out_dtype, "many rows")
    assert torch.equal(whole_h.cpu(), h + delta.float())
    for first in (0, 100, 505):
        part_h = h[first:first + 10].to(DEV)
        part = F().add_rmsnorm(part_h, delta[first:first + 10].to(DEV), w.to(DEV), eps, out_dtype)
        assert torch.equal(part.cpu(), whole.cpu()[first:first + 10])
        assert torch.equal(part_h.cpu(), whole_h.cpu()[first:first + 10])
    rows = torch.arange(n - 1, -1, -1, dtype=torch.int32)
    untouched = h.to(DEV)
    picked = F().add_rmsnorm(untouched, delta.to(DEV), w.to(DEV), eps, out_dtype, rows=rows.to(DEV))
    assert torch.equal(picked.cpu(), whole.cpu().flip(0)) and torch.equal(untouched.cpu(), h)
    alone = F().add_rmsnorm(h.to(DEV), None, w.to(DEV), eps, out_dtype)
    close(alone, plain.rms_norm(h.double(), w.double(), eps), out_dtype, "many rows without delta")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    n, inter = 5, 224 + 3
    gu = rand(n, 2 * inter, seed=4, scale=3.0).to(dtype)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    close(F().swiglu(gu.to(DEV)), g * torch.sigmoid(g) * u, dtype, "swiglu")


def scrambled_pages(n_seqs, max_len, n_kv, d, dtype, seed=0, page=64, extra=3):
    """A PagedKV whose pages are handed out in random order, every place poisoned with NaN."""
    per_seq = -(-max_len // page)
    n_pages = n_seqs * per_seq + extra
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))
    table = torch.full((n_seqs + 2, per_seq), -1, dtype=torch.int32)
    slots = torch.randperm(n_seqs + 2, generator=torch.Generator().manual_seed(seed + 1))[:n_seqs].to(torch.int32)
    for i in range(n_seqs):
        table[slots[i]] = perm[i * per_seq:(i + 1) * per_seq].to(torch.int32)
    k = torch.full((n_pages, n_kv, page, d), float("nan"), dtype=dtype)
    v = torch.full((n_pages, n_kv, page, d), float("nan"), dtype=dtype)
    return F().PagedKV(k.to(DEV), v.to(DEV), table.clamp(min=0).to(DEV)), slots, table


def fill_pages(kv, table, slot, keys, values):
    """Writes a sequence's keys and values [len, n_kv, d] into its pages (test-side, with torch)."""
    page = kv.page_size
    for start in range(0, keys.shape[0], page):
        p = int(table[slot, start // page])
        n = min(page, keys.shape[0] - start)
        kv.k[p, :, :n] = keys[start:start + n].transpose(0, 1).to(kv.k.dtype).to(DEV)
        kv.v[p, :, :n] = values[start:start + n].transpose(0, 1).to(kv.v.dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,theta", [(6, 3, 48, 1e4), (4, 1, 128, 1e6), (5, 5, 16, 5e5)])
def test_qk_norm_rope_write(dtype, n_q, n_kv, d, theta):
    eps = 2e-6
    lens = [70, 1, 130]
    past = [60, 0, 3]  # tokens already cached; the step brings the rest
    kv, slots, table = scrambled_pages(3, 130, n_kv, d, dtype, seed=5)
    width = (n_q + 2 * n_kv) * d
    rows, pos, seq = [], [], []
    for i, (n, p) in enumerate(zip(lens, past)):
        rows.append(rand(n - p, width, seed=10 + i).to(dtype))
        pos += list(range(p, n))
        seq += [i] * (n - p)
    qkv = torch.cat(rows)
    wq = (1 + 0.1 * rand(d, seed=20)).float()
    wk = (1 + 0.1 * rand(d, seed=21)).float()
    cos, sin = plain.rotary_tables(torch.arange(131), d, theta)
    tok_pos = torch.tensor(pos, dtype=torch.int32)
    q = F().qk_norm_rope_write(
        qkv.to(DEV), n_q, n_kv, d, wq.to(DEV), wk.to(DEV), eps, cos[:, : d // 2].contiguous().to(DEV),
        sin[:, : d // 2].contiguous().to(DEV), tok_pos.to(DEV), torch.tensor(seq, dtype=torch.int32).to(DEV),
        slots.to(DEV), kv, max(pos))
    x = qkv.double().view(-1, n_q + 2 * n_kv, d)
    c, s = cos[tok_pos.long()].double(), sin[tok_pos.long()].double()
    want_q = plain.apply_rotary(plain.rms_norm(x[:, :n_q], wq.double(), eps), c, s)
    want_k = plain.apply_rotary(plain.rms_norm(x[:, n_q:n_q + n_kv], wk.double(), eps), c, s)
    want_v = x[:, n_q + n_kv:]
    close(q, want_q, dtype, "q")
    written = torch.zeros(kv.k.shape[0], kv.page_size, dtype=torch.bool)
    for t, (p, i) in enumerate(zip(pos, seq)):
        page = int(table[slots[i], p // 64])
        close(kv.k[page, :, p % 64], want_k[t], dtype, f"k of token {t}")
        close(kv.v[page, :, p % 64], want_v[t], dtype, f"v of token {t}", atol=1e-7)
        written[page, p % 64] = True
    # nothing else was written: every other place still holds its poison
    assert torch.isnan(kv.k.cpu().float()[~written[:, None, :].expand(-1, n_kv, -1)]).all()


def test_qk_write_without_norm_or_rotation_and_read_only():
    n_q, n_kv, d = 2, 2, 32
    kv, slots, table = scrambled_pages(1, 10, n_kv, d, torch.float32)
    qkv = rand(10, (n_q + 2 * n_kv) * d).float()
    ids = torch.arange(10, dtype=torch.int32).to(DEV)
    zeros = torch.zeros(10, dtype=torch.int32).to(DEV)
    q = F().qk_norm_rope_write(qkv.to(DEV), n_q, n_kv, d, None, None, 1.0, None, None, ids, zeros, slots.to(DEV), kv, 9,
                               write_kv=False)
    assert torch.equal(q.cpu().view(10, -1), qkv[:, : n_q * d]) and torch.isnan(kv.k).all()
    F().qk_norm_rope_write(qkv.to(DEV), n_q, n_kv, d, None, None, 1.0, None, None, ids, zeros, slots.to(DEV), kv, 9)
    page = int(table[slots[0], 0])
    assert torch.equal(kv.k[page, :, :10].cpu().transpose(0, 1).reshape(10, -1), qkv[:, n_q * d:(n_q + n_kv) * d])


# ------------------------------------------------------------------ 32-bit matrix product
@pytest.mark.parametrize("m,n,k", [(1, 71, 53), (37, 300, 1000), (130, 129, 257), (64, 1000, 7)])
@pytest.mark.parametrize("a_dtype,c_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_gemm_f32_is_true_32_bit(m, n, k, a_dtype, c_dtype):
    a = rand(m, k, seed=1).to(a_dtype)
    w = rand(n, k, seed=2).float()
    got = F().linear_f32(a.to(DEV), w.to(DEV), c_dtype)
    want = a.double() @ w.double().T
    if c_dtype == torch.float32:
        # TF32 or bfloat16 products would miss by ~1e-3 * sqrt(k); float32 chains stay near 1e-6 * sqrt(k)
        err = (got.double().cpu() - want).abs().max().item()
        assert err < 2e-6 * math.sqrt(k) * 4, f"{err:.3e}"
    else:
        close(got, want, c_dtype, "gemm bf16 out")


def test_gemm_f32_rows_do_not_depend_on_the_batch():
    a = rand(200, 333, seed=3).float().to(DEV)
    w = rand(150, 333, seed=4).float().to(DEV)
    whole = F().linear_f32(a, w)
    for start, stop in ((0, 1), (7, 8), (100, 164), (199, 200)):
        assert torch.equal(F().linear_f32(a[start:stop].contiguous(), w), whole[start:stop])


# ------------------------------------------------------------------ attention
def dense_attention(q, k, v, past, window=None):
    """Plain attention of the last len(q) positions of one sequence: q [T, n_q, d], k/v [S, n_kv, d]."""
    n_kv = k.shape[1]
    full_q = torch.zeros(k.shape[0], q.shape[1], q.shape[2], dtype=torch.float64)
    full_q[past:] = q
    return plain.causal_gqa_attention(full_q, k, v, window)[past:]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d", [(4, 4, 16), (4, 2, 48), (6, 2, 80), (8, 2, 128)])
def test_attention_exact_varlen(dtype, n_q, n_kv, d):
    lens, past = [1, 777, 1000, 64], [0, 700, 999, 0]  # whole prompts, a continuation, a decode step
    kv, slots, table = scrambled_pages(4, 1000, n_kv, d, dtype, seed=8)
    qs, pos, seq, wants = [], [], [], []
    for i, (n, p) in enumerate(zip(lens, past)):
        k = rand(n, n_kv, d, seed=30 + i).to(dtype)
        v = rand(n, n_kv, d, seed=40 + i).to(dtype)
        q = rand(n - p, n_q, d, seed=50 + i).to(dtype)
        fill_pages(kv, table, int(slots[i]), k, v)
        qs.append(q)
        pos += list(range(p, n))
        seq += [i] * (n - p)
        wants.append(dense_attention(q.double(), k.double(), v.double(), p))
    out = F().attention_exact(torch.cat(qs).to(DEV), kv, torch.tensor(pos, dtype=torch.int32).to(DEV),
                              torch.tensor(seq, dtype=torch.int32).to(DEV), slots.to(DEV), d**-0.5)
    want = torch.cat(wants)
    got = out.double().cpu()
    assert torch.isfinite(got).all()  # no poisoned place was read
    tol = 2e-5 if dtype == torch.float32 else 1.5 * BF16_ULP * want.abs().max().item() + 1e-3
    assert (got - want).abs().max().item() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    n_q, n_kv, d, n = 4, 2, 64, 900
    kv, slots, table = scrambled_pages(1, n, n_kv, d, dtype, seed=9)
    k = rand(n, n_kv, d, seed=1, scale=0.1)
    v = rand(n, n_kv, d, seed=2)
    q = rand(1, n_q, d, seed=3, scale=0.1)
    far = {0: 3, 1: 517}  # kv head -> the key that must win, one near the start, one deep inside
    for hk, j in far.items():
        direction = torch.ones(d, dtype=torch.float64)
        k[j, hk] = 6.0 * direction
        q[0, 2 * hk] = 6.0 * direction  # query heads 0 and 2: score 36*64/8 = 288 against O(1) elsewhere
    fill_pages(kv, table, int(slots[0]), k.to(dtype), v.to(dtype))
    out = F().attention_exact(q.to(dtype).to(DEV), kv, torch.tensor([n - 1], dtype=torch.int32).to(DEV),
                              torch.zeros(1, dtype=torch.int32).to(DEV), slots.to(DEV), d**-0.5).double().cpu()
    for hk, j in far.items():
        assert (out[0, 2 * hk] - v[j, hk].to(dtype).double()).abs().max() < 1e-5, f"kv head {hk}: key {j} was not found"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_window_edge(dtype):
    n_q, n_kv, d, n, window = 2, 1, 32, 300, 100
    kv, slots, table = scrambled_pages(1, n, n_kv, d, dtype, seed=10)
    k = rand(n, n_kv, d, seed=1, scale=0.1)
    v = rand(n, n_kv, d, seed=2)
    q = rand(1, n_q, d, seed=3, scale=0.1)
    pos = n - 1
    inside, outside = pos - window + 1, pos - window  # the last key inside the window, the first outside
    k[inside, 0] = 4.0
    k[outside, 0] = 8.0  # would win by far if it were visible
    q[0, :] = 4.0
    fill_pages(kv, table, int(slots[0]), k.to(dtype), v.to(dtype))
    args = (q.to(dtype).to(DEV), kv, torch.tensor([pos], dtype=torch.int32).to(DEV),
            torch.zeros(1, dtype=torch.int32).to(DEV), slots.to(DEV), d**-0.5)
    out = F().attention_exact(*args, window=window).double().cpu()
    assert (out[0, 0] - v[inside, 0].to(dtype).double()).abs().max() < 1e-5
    out_all = F().attention_exact(*args, window=0).double().cpu()
    assert (out_all[0, 0] - v[outside, 0].to(dtype).double()).abs().max() < 1e-5
    want = dense_attention(q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double(), pos, window)
    assert (out - want).abs().max() < (2e-5 if dtype == torch.float32 else 2e-2)


def test_attention_exact_is_the_same_for_any_cut():
    n_q, n_kv, d, n = 4, 2, 48, 200
    kv, slots, table = scrambled_pages(1, n, n_kv, d, torch.float32, seed=11)
    fill_pages(kv, table, int(slots[0]), rand(n, n_kv, d, seed=1).float(), rand(n, n_kv, d, seed=2).float())
    q = rand(n, n_q, d, seed=3).float().to(DEV)
    zeros = torch.zeros(n, dtype=torch.int32).to(DEV)
    pos = torch.arange(n, dtype=torch.int32).to(DEV)
    whole = F().attention_exact(q, kv, pos, zeros, slots.to(DEV), d**-0.5)
    for t in (0, 31, 32, 63, 64, 199):
        one = F().attention_exact(q[t:t + 1].contiguous(), kv, pos[t:t + 1].contiguous(), zeros[:1].contiguous(),
                                  slots.to(DEV), d**-0.5)
        assert torch.equal(one[0], whole[t])


# ------------------------------------------------------------------ token choice
@pytest.mark.parametrize("vocab", [384, 1000 + 7, 151936])
def test_argmax_lowest_index_wins(vocab):
    logits = rand(5, vocab, seed=1).float()
    logits[1, 17] = logits[1, vocab - 1] = 50.0
    logits[2, vocab - 1] = 60.0
    logits[3, 0] = 60.0
    logits[4] = -3.0  # all equal
    got = F().argmax(logits.to(DEV)).cpu().tolist()
    assert got == [int(logits[0].argmax()), 17, vocab - 1, 0, 0]


@pytest.mark.parametrize("vocab,top_k", [(384, 0), (1007, 50), (1007, 1), (151936, 50), (4000, 5000)])
def test_sample_matches_the_plain_sampler(vocab, top_k):
    n, seed, temperature = 6, 1234, 0.8
    logits = rand(n, vocab, seed=2, scale=2.0).float()
    if top_k:
        logits[0, :100] = logits[0, 0]  # a hundred-way tie around the threshold
    requests = torch.tensor([0, 1, 2, 77, 4, 5], dtype=torch.int32)
    steps = torch.tensor([0, 0, 9, 3, 100000, 1], dtype=torch.int32)
    steps_dev = steps.to(DEV)
    got = F().sample(logits.to(DEV), temperature, top_k, seed, requests.to(DEV), steps_dev, advance_steps=True).cpu().tolist()
    want = [plain_sampling.sample(logits[i].numpy(), temperature, top_k, seed, int(requests[i]), int(steps[i]))
            for i in range(n)]
    assert got == want
    assert torch.equal(steps_dev.cpu(), steps + 1)


@pytest.mark.parametrize("n", [40, 100, 400])
def test_sample_and_argmax_with_many_rows(n):
    """The number of blocks that share a row falls as the rows grow (eight, four, two, one for the top-k
    threshold); the choice must not depend on it."""
    vocab, top_k, seed, temperature = 5003, 7, 99, 1.3
    logits = rand(n, vocab, seed=3, scale=2.0).float()
    requests = torch.arange(n, dtype=torch.int32)
    steps = (torch.arange(n, dtype=torch.int32) * 7) % 13
    got = F().sample(logits.to(DEV), temperature, top_k, seed, requests.to(DEV), steps.to(DEV)).cpu().tolist()
    want = [plain_sampling.sample(logits[i].numpy(), temperature, top_k, seed, int(requests[i]), int(steps[i])) for i in range(n)]
    assert got == want
    assert F().argmax(logits.to(DEV)).cpu().tolist() == logits.argmax(-1).tolist()


def test_sample_follows_the_softmax():
    logits = torch.tensor([[1.0, 0.0, -1.0, 2.0, 0.5]]).repeat(4096, 1)
    z = logits[0].double() / 0.7
    p = torch.softmax(z, 0)
    counts = torch.zeros(5)
    requests = torch.arange(4096, dtype=torch.int32).to(DEV)
    for step in range(4):
        steps = torch.full((4096,), step, dtype=torch.int32).to(DEV)
        tokens = F().sample(logits.to(DEV), 0.7, 0, 9, requests, steps).cpu()
        counts += torch.bincount(tokens.long(), minlength=5)
    assert (counts / counts.sum() - p).abs().max() < 0.015


# ------------------------------------------------------------------ bfloat16 decode attention (split-KV)
@pytest.mark.parametrize("n_q,n_kv,d", [(4, 4, 64), (16, 8, 128), (6, 2, 128), (16, 1, 64)])
@pytest.mark.parametrize("n_splits,use_scratch", [(1, False), (3, False), (8, False), (3, True), (40, False)])
def test_attention_decode_bf16(n_q, n_kv, d, n_splits, use_scratch):
    dtype = torch.bfloat16
    lens = [1, 63, 64, 65, 777, 1000, 130]
    kv, slots, table = scrambled_pages(len(lens), 1000, n_kv, d, dtype, seed=12)
    qs, wants = [], []
    for i, n in enumerate(lens):
        k = rand(n, n_kv, d, seed=60 + i).to(dtype)
        v = rand(n, n_kv, d, seed=70 + i).to(dtype)
        q = rand(1, n_q, d, seed=80 + i).to(dtype)
        fill_pages(kv, table, int(slots[i]), k, v)
        qs.append(q)
        wants.append(dense_attention(q.double(), k.double(), v.double(), n - 1))
    kv_len = torch.tensor(lens, dtype=torch.int32).to(DEV)
    out = F().attention_decode(torch.cat(qs).to(DEV), kv, kv_len, slots.to(DEV), d**-0.5, 0, n_splits, use_scratch=use_scratch)
    got, want = out.double().cpu(), torch.cat(wants)
    assert torch.isfinite(got).all()  # the poisoned places beyond each length were not used
    # the yardstick: the exact kernel on the same bfloat16 inputs rounds its output once
    assert (got - want).abs().max().item() < 1.5 * BF16_ULP * want.abs().max().item() + 2e-3


def test_attention_decode_bf16_far_key_and_window():
    dtype, n_q, n_kv, d, n = torch.bfloat16, 8, 2, 128, 900
    kv, slots, table = scrambled_pages(1, n, n_kv, d, dtype, seed=13)
    k = rand(n, n_kv, d, seed=1, scale=0.1)
    v = rand(n, n_kv, d, seed=2)
    q = rand(1, n_q, d, seed=3, scale=0.1)
    k[5, 0] = 3.0
    q[0, 1] = 3.0   # query head 1 (kv head 0) must find key 5: score 9*128/sqrt(128) = 102
    k[517, 1] = 3.0
    q[0, 6] = 3.0   # query head 6 (kv head 1) must find key 517
    fill_pages(kv, table, int(slots[0]), k.to(dtype), v.to(dtype))
    kv_len = torch.tensor([n], dtype=torch.int32).to(DEV)
    for splits in (1, 7):
        out = F().attention_decode(q.to(dtype).to(DEV), kv, kv_len, slots.to(DEV), d**-0.5, 0, splits).double().cpu()
        assert (out[0, 1] - v[5, 0].to(dtype).double()).abs().max() < 1e-2
        assert (out[0, 6] - v[517, 1].to(dtype).double()).abs().max() < 1e-2
        # a window of 400 hides key 5 (visible keys are 500..899) but not key 517
        win = F().attention_decode(q.to(dtype).to(DEV), kv, kv_len, slots.to(DEV), d**-0.5, 400, splits).double().cpu()
        want = dense_attention(q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double(), n - 1, 400)
        assert (win - want).abs().max() < 2e-2
        assert (win[0, 1] - v[5, 0].to(dtype).double()).abs().max() > 0.1
        # the key at the window's edge: 500 is the last one inside, 499 the first outside
        k2 = k.clone()
        k2[499, 0] = 6.0
        k2[500, 0] = 3.0
        k2[5, 0] = 0.0
        fill_pages(kv, table, int(slots[0]), k2.to(dtype), v.to(dtype))
        edge = F().attention_decode(q.to(dtype).to(DEV), kv, kv_len, slots.to(DEV), d**-0.5, 400, splits).double().cpu()
        assert (edge[0, 1] - v[500, 0].to(dtype).double()).abs().max() < 1e-2
        fill_pages(kv, table, int(slots[0]), k.to(dtype), v.to(dtype))


@pytest.mark.parametrize("n_q,n_kv,d", [(4, 4, 64), (16, 8, 128), (6, 2, 128), (16, 1, 64), (12, 3, 128)])
@pytest.mark.parametrize("n_blocks", [1, 2, 7, 64, 0, 1000])
def test_attention_decode_dealt_evenly(n_q, n_kv, d, n_blocks):
    """The kernel that cuts the line of all sequences' pages into equal pieces: pieces that end inside a pair, pairs
    spread over many blocks, more blocks than pages; twice in a row, since the ticket counters must be left at zero."""
    dtype = torch.bfloat16
    lens = [1, 63, 64, 65, 777, 1000, 130, 2, 128]
    kv, slots, table = scrambled_pages(len(lens), 1000, n_kv, d, dtype, seed=12)
    kv.work = F().DecodeWork(torch.device(DEV))
    qs, wants = [], []
    for i, n in enumerate(lens):
        k = rand(n, n_kv, d, seed=60 + i).to(dtype)
        v = rand(n, n_kv, d, seed=70 + i).to(dtype)
        q = rand(1, n_q, d, seed=80 + i).to(dtype)
        fill_pages(kv, table, int(slots[i]), k, v)
        qs.append(q)
        wants.append(dense_attention(q.double(), k.double(), v.double(), n - 1))
    kv_len = torch.tensor(lens, dtype=torch.int32).to(DEV)
    want = torch.cat(wants)
    for turn in range(2):
        out = F().attention_decode_flat(torch.cat(qs).to(DEV), None, n_q, n_kv, d, None, None, 1.0, None, None, kv, kv_len,
                                        slots.to(DEV), max(lens) - 1, d**-0.5, 0, n_blocks)
        got = out.double().cpu()
        assert torch.isfinite(got).all()  # the poisoned places beyond each length were not used
        assert (got - want).abs().max().item() < 1.5 * BF16_ULP * want.abs().max().item() + 2e-3, turn
        assert int(kv.work.tickets.abs().sum()) == 0


def test_attention_decode_dealt_evenly_far_key_and_window():
    dtype, n_q, n_kv, d, n = torch.bfloat16, 8, 2, 128, 900
    kv, slots, table = scrambled_pages(1, n, n_kv, d, dtype, seed=13)
    k = rand(n, n_kv, d, seed=1, scale=0.1)
    v = rand(n, n_kv, d, seed=2)
    q = rand(1, n_q, d, seed=3, scale=0.1)
    k[5, 0] = 3.0
    q[0, 1] = 3.0   # query head 1 (kv head 0) must find key 5
    k[517, 1] = 3.0
    q[0, 6] = 3.0   # query head 6 (kv head 1) must find key 517
    fill_pages(kv, table, int(slots[0]), k.to(dtype), v.to(dtype))
    kv_len = torch.tensor([n], dtype=torch.int32).to(DEV)

    def run(window, blocks):
        return F().attention_decode_flat(q.to(dtype).to(DEV), None, n_q, n_kv, d, None, None, 1.0, None, None, kv, kv_len,
                                         slots.to(DEV), n - 1, d**-0.5, window, blocks).double().cpu()

    for blocks in (1, 5, 0):
        out = run(0, blocks)
        assert (out[0, 1] - v[5, 0].to(dtype).double()).abs().max() < 1e-2
        assert (out[0, 6] - v[517, 1].to(dtype).double()).abs().max() < 1e-2
        # a window of 400 hides key 5 (visible keys are 500..899) but not key 517
        win = run(400, blocks)
        want = dense_attention(q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double(), n - 1, 400)
        assert (win - want).abs().max() < 2e-2
        assert (win[0, 1] - v[5, 0].to(dtype).double()).abs().max() > 0.1
        # the key at the window's edge: 500 is the last one inside, 499 the first outside
        k2 = k.clone()
        k2[499, 0] = 6.0
        k2[500, 0] = 3.0
        k2[5, 0] = 0.0
        fill_pages(kv, table, int(slots[0]), k2.to(dtype), v.to(dtype))
        edge = run(400, blocks)
        assert (edge[0, 1] - v[500, 0].to(dtype).double()).abs().max() < 1e-2
        fill_pages(kv, table, int(slots[0]), k.to(dtype), v.to(dtype))


# ------------------------------------------------------------------ tcgen05 matrix product
@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (8, 256, 128), (8, 4096, 1024), (13, 1000, 200), (64, 384, 1024),
                                   (65, 128, 64), (128, 128, 128), (200, 1000, 520), (2048, 1024, 3072), (300, 151936, 1024),
                                   (203, 1008, 520)])  # the last: rows end inside a quad of lanes, columns inside a tile
def test_gemm_tc_plain(m, n, k):
    x = rand(m, k, seed=1).to(torch.bfloat16)
    w = rand(n, k, seed=2, scale=0.05).to(torch.bfloat16)
    if n > 100000:  # compare a slice of the very wide case on the host
        got = F().gemm_tc(x.to(DEV), w.to(DEV), torch.float32)
        F().check_kernel_errors()
        cols = torch.cat([torch.arange(0, 300), torch.arange(n - 300, n), torch.arange(70000, 70300)])
        want = x.double() @ w.double()[cols].T
        assert (got.cpu().double()[:, cols] - want).abs().max() < 1e-3 * (k ** 0.5)
        return
    want = x.double() @ w.double().T
    for out_dtype in (torch.bfloat16, torch.float32):
        got = F().gemm_tc(x.to(DEV), w.to(DEV), out_dtype)
        F().check_kernel_errors()
        err = (got.cpu().double() - want).abs().max().item()
        bound = 2e-5 * (k ** 0.5) if out_dtype == torch.float32 else BF16_ULP * want.abs().max().item() + 1e-4
        assert err < bound, f"{out_dtype}: {err:.3e} >= {bound:.3e}"


@pytest.mark.parametrize("m,n,k,splits", [(8, 1024, 2048, 8), (3, 256, 192, 2), (64, 1024, 3072, 4), (8, 128, 64, 4), (33, 1000, 1024, 8)])
def test_gemm_tc_split_k(m, n, k, splits):
    x = rand(m, k, seed=3).to(torch.bfloat16)
    w = rand(n, k, seed=4, scale=0.05).to(torch.bfloat16)
    want = x.double() @ w.double().T
    first = None
    for _ in range(3):  # the counters must be back at zero after every launch
        got = F().gemm_tc(x.to(DEV), w.to(DEV), torch.float32, splits=splits)
        F().check_kernel_errors()
        assert got.shape == (m, n)
        assert (got.cpu().double() - want).abs().max() < 2e-5 * (k ** 0.5)
        first = got if first is None else first
        assert torch.equal(got, first)  # summed in split order: the same bits every time


@pytest.mark.parametrize("m,inter,k,splits", [(8, 3072, 1024, 1), (8, 3072, 1024, 2), (5, 100, 72, 1), (64, 224, 80, 2),
                                               (300, 224, 136, 1), (2048, 3072, 1024, 1), (203, 528, 136, 1)])
def test_gemm_tc_swiglu(m, inter, k, splits):
    x = rand(m, k, seed=5).to(torch.bfloat16)
    gate = rand(inter, k, seed=6, scale=0.1).to(torch.bfloat16)
    up = rand(inter, k, seed=7, scale=0.1).to(torch.bfloat16)
    packed = torch.stack([gate, up], dim=1).reshape(2 * inter, k).contiguous()  # gate0, up0, gate1, up1, ...
    got = F().gemm_tc(x.to(DEV), packed.to(DEV), swiglu=True, splits=splits)
    F().check_kernel_errors()
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    want = g * torch.sigmoid(g) * u
    assert got.shape == (m, inter)
    assert (got.cpu().double() - want).abs().max() < BF16_ULP * want.abs().max().item() + 1e-3


def test_swiglu_interleaved():
    gu = rand(3, 2 * 50, seed=8, scale=2.0).float()
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()
    close(F().swiglu(gu.to(DEV), interleaved=True), g * torch.sigmoid(g) * u, torch.float32, "interleaved swiglu")


# ------------------------------------------------------------------ bfloat16 flash prefill attention
def prefill_attention(path, *args, **kwargs):
    """``path``: "mma", "tcgen05_128", "tcgen05_64" (the tcgen05 kernels with 128 or 64 keys per step) or
    "tcgen05_128_pairs" (128 keys per step, a heavy and a light query tile a block instead of a tile a block), or
    "tcgen05_128_stay" (128 keys per step, blocks that stay and take tiles from a list)."""
    if not path.startswith("tcgen05_"):
        return F().attention_prefill(*args, tensor_cores=path, **kwargs)
    before = F().set_attention_prefill_keys(int(path[8:].split("_")[0]))
    one = F().set_attention_prefill_one_tile(0 if path.endswith("_pairs") else 1)
    stay = F().set_attention_prefill_stay(1 if path.endswith("_stay") else 0)
    try:
        return F().attention_prefill(*args, tensor_cores="tcgen05", **kwargs)
    finally:
        F().set_attention_prefill_keys(before)
        F().set_attention_prefill_one_tile(one)
        F().set_attention_prefill_stay(stay)


@pytest.mark.parametrize("n_q,n_kv,d,path", [(4, 4, 64, "mma"), (16, 8, 128, "mma"), (6, 2, 128, "mma"), (3, 1, 64, "mma"),
                                              (16, 8, 128, "tcgen05_128"), (6, 2, 128, "tcgen05_128"), (4, 4, 128, "tcgen05_128"),
                                              (16, 8, 128, "tcgen05_64"), (6, 2, 128, "tcgen05_64"), (4, 4, 128, "tcgen05_64"),
                                              (16, 8, 128, "tcgen05_128_pairs"), (6, 2, 128, "tcgen05_128_pairs"), (4, 4, 128, "tcgen05_128_pairs"),
                                              (16, 8, 128, "tcgen05_128_stay"), (8, 2, 128, "tcgen05_128_stay"), (4, 4, 128, "tcgen05_128_stay")])
def test_attention_prefill_bf16_varlen(n_q, n_kv, d, path):
    dtype = torch.bfloat16
    lens, past = [1, 777, 1000, 64, 130], [0, 700, 0, 0, 129]  # whole prompts, a continuation, a single token
    kv, slots, table = scrambled_pages(len(lens), 1000, n_kv, d, dtype, seed=14)
    qs, wants, cu = [], [], [0]
    for i, (n, p) in enumerate(zip(lens, past)):
        k = rand(n, n_kv, d, seed=90 + i).to(dtype)
        v = rand(n, n_kv, d, seed=100 + i).to(dtype)
        q = rand(n - p, n_q, d, seed=110 + i).to(dtype)
        fill_pages(kv, table, int(slots[i]), k, v)
        qs.append(q)
        cu.append(cu[-1] + n - p)
        wants.append(dense_attention(q.double(), k.double(), v.double(), p))
    out = prefill_attention(path, torch.cat(qs).to(DEV), kv, torch.tensor(cu, dtype=torch.int32).to(DEV),
                            torch.tensor(lens, dtype=torch.int32).to(DEV), slots.to(DEV),
                            max(n - p for n, p in zip(lens, past)), d**-0.5)
    F().check_kernel_errors()
    got, want = out.double().cpu(), torch.cat(wants)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() < 1.5 * BF16_ULP * want.abs().max().item() + 2e-3


@pytest.mark.parametrize("path", ["mma", "tcgen05_128", "tcgen05_64", "tcgen05_128_pairs", "tcgen05_128_stay"])
def test_attention_prefill_bf16_far_key_and_window(path):
    dtype, n_q, n_kv, d, n = torch.bfloat16, 4, 2, 128, 900
    kv, slots, table = scrambled_pages(1, n, n_kv, d, dtype, seed=15)
    k = rand(n, n_kv, d, seed=1, scale=0.1)
    v = rand(n, n_kv, d, seed=2)
    q = rand(n, n_q, d, seed=3, scale=0.1)
    k[5, 0] = 3.0
    q[700:, 1] = 3.0  # head 1 (kv head 0) of the late tokens must find key 5 among hundreds
    fill_pages(kv, table, int(slots[0]), k.to(dtype), v.to(dtype))
    args = (q.to(dtype).to(DEV), kv, torch.tensor([0, n], dtype=torch.int32).to(DEV), torch.tensor([n], dtype=torch.int32).to(DEV),
            slots.to(DEV), n, d**-0.5)
    out = prefill_attention(path, *args).double().cpu()
    F().check_kernel_errors()
    assert (out[700:, 1] - v[5, 0].to(dtype).double()).abs().max() < 1e-2
    want = dense_attention(q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double(), 0)
    assert (out - want).abs().max() < 2e-2
    win = prefill_attention(path, *args, window=100).double().cpu()
    want_w = dense_attention(q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double(), 0, 100)
    assert (win - want_w).abs().max() < 2e-2
    assert (win[700:, 1] - v[5, 0].to(dtype).double()).abs().max() > 0.1  # key 5 is outside every late token's window


# ------------------------------------------------------------------ decode attention fused with norm, rotation and cache write
@pytest.mark.parametrize("n_q,n_kv,d,weight_dtype", [(16, 8, 128, torch.float32), (4, 1, 64, torch.float32), (6, 2, 128, torch.bfloat16)])
@pytest.mark.parametrize("n_splits", [1, 4])
def test_attention_decode_fused_equals_the_separate_kernels(n_q, n_kv, d, weight_dtype, n_splits):
    dtype, eps, theta = torch.bfloat16, 1e-6, 1e6
    lens = [1, 64, 65, 300, 1000]  # the new token is the last of each: at a page's first, last and inner places
    width = (n_q + 2 * n_kv) * d
    qkv = rand(len(lens), width, seed=1).to(dtype)
    wq, wk = (1 + 0.1 * rand(d, seed=2)).to(weight_dtype), (1 + 0.1 * rand(d, seed=3)).to(weight_dtype)
    cos, sin = plain.rotary_tables(torch.arange(1001), d, theta)
    cos, sin = cos[:, : d // 2].contiguous().to(DEV), sin[:, : d // 2].contiguous().to(DEV)
    kv_len = torch.tensor(lens, dtype=torch.int32).to(DEV)
    results = []
    for fused in (False, True, "dealt evenly", "dealt evenly, three blocks"):
        kv, slots, table = scrambled_pages(len(lens), 1000, n_kv, d, dtype, seed=16)
        for i, n in enumerate(lens):  # the cached past of each sequence (everything but the new token)
            if n > 1:
                fill_pages(kv, table, int(slots[i]), rand(n - 1, n_kv, d, seed=20 + i).to(dtype), rand(n - 1, n_kv, d, seed=30 + i).to(dtype))
        pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32).to(DEV)
        seq = torch.arange(len(lens), dtype=torch.int32).to(DEV)
        if isinstance(fused, str):
            out = F().attention_decode_flat(None, qkv.to(DEV), n_q, n_kv, d, wq.to(DEV), wk.to(DEV), eps, cos, sin, kv, kv_len,
                                            slots.to(DEV), max(lens) - 1, d**-0.5, 0, 3 if "three" in fused else 0)
        elif fused:
            out = F().attention_decode_fused(qkv.to(DEV), n_q, n_kv, d, wq.to(DEV), wk.to(DEV), eps, cos, sin, kv, kv_len,
                                             slots.to(DEV), max(lens) - 1, d**-0.5, 0, n_splits)
        else:
            q = F().qk_norm_rope_write(qkv.to(DEV), n_q, n_kv, d, wq.to(DEV), wk.to(DEV), eps, cos, sin, pos, seq, slots.to(DEV),
                                       kv, max(lens) - 1)
            out = F().attention_decode(q, kv, kv_len, slots.to(DEV), d**-0.5, 0, n_splits)
        new_k = torch.stack([kv.k[int(table[slots[i], (n - 1) // 64]), :, (n - 1) % 64] for i, n in enumerate(lens)])
        new_v = torch.stack([kv.v[int(table[slots[i], (n - 1) // 64]), :, (n - 1) % 64] for i, n in enumerate(lens)])
        results.append((out.float().cpu(), new_k.float().cpu(), new_v.float().cpu()))
    out_a, k_a, v_a = results[0]
    for out_b, k_b, v_b in results[1:]:
        assert torch.isfinite(out_b).all()
        assert torch.equal(v_a, v_b)
        # the same formulas in the same precision; the fused kernels may contract a multiply-add differently
        assert (k_a - k_b).abs().max() <= 2.0**-7 * k_a.abs().max()
        assert (out_a - out_b).abs().max() <= 2.0**-7 * out_a.abs().max() + 1e-3


# ------------------------------------------------------------------ q|k|v projection with the attention input stage in its epilogue
@pytest.mark.parametrize("n_q,n_kv,d,hidden,weight_dtype", [(16, 8, 128, 1024, torch.float32), (6, 2, 64, 136, torch.bfloat16),
                                                            (5, 1, 128, 72, torch.float32)])
def test_gemm_tc_qkv_equals_projection_then_qk_kernel(n_q, n_kv, d, hidden, weight_dtype):
    dtype, eps, theta = torch.bfloat16, 1e-6, 1e5
    lens, past = [700, 1300, 60], [0, 300, 59]
    n_tokens = sum(n - p for n, p in zip(lens, past))
    width = (n_q + 2 * n_kv) * d
    x = rand(n_tokens, hidden, seed=1).to(dtype)
    w = rand(width, hidden, seed=2, scale=hidden**-0.5).to(dtype)
    wq, wk = (1 + 0.1 * rand(d, seed=3)).to(weight_dtype), (1 + 0.1 * rand(d, seed=4)).to(weight_dtype)
    cos, sin = plain.rotary_tables(torch.arange(1301), d, theta)
    cos, sin = cos[:, : d // 2].contiguous().to(DEV), sin[:, : d // 2].contiguous().to(DEV)
    pos, seq = [], []
    for i, (n, p) in enumerate(zip(lens, past)):
        pos += list(range(p, n))
        seq += [i] * (n - p)
    pos_d, seq_d = torch.tensor(pos, dtype=torch.int32).to(DEV), torch.tensor(seq, dtype=torch.int32).to(DEV)
    results = []
    for fused in (False, True):
        kv, slots, table = scrambled_pages(3, 1300, n_kv, d, dtype, seed=17)
        if fused:
            assert F().qkv_fused_ok(x.to(DEV), w.to(DEV), d, kv) == (n_q == 16)  # the engine fuses only wide products
            q = F().gemm_tc_qkv(x.to(DEV), w.to(DEV), n_q, n_kv, d, wq.to(DEV), wk.to(DEV), eps, cos, sin, pos_d, seq_d,
                                slots.to(DEV), kv, max(pos))
        else:
            qkv = F().gemm_tc(x.to(DEV), w.to(DEV))
            q = F().qk_norm_rope_write(qkv, n_q, n_kv, d, wq.to(DEV), wk.to(DEV), eps, cos, sin, pos_d, seq_d, slots.to(DEV), kv, max(pos))
        F().check_kernel_errors()
        results.append((q.float().cpu(), kv.k.float().cpu(), kv.v.float().cpu()))
    (q_a, k_a, v_a), (q_b, k_b, v_b) = results
    assert torch.isfinite(q_b).all()
    written = ~torch.isnan(k_a)
    assert torch.equal(written, ~torch.isnan(k_b)) and torch.equal(~torch.isnan(v_a), ~torch.isnan(v_b))  # the same places
    # the unfused path rounds the projection to bfloat16 before the norm, the fused one does not
    assert (q_a - q_b).abs().max() <= 2.0**-6 * q_a.abs().max()
    assert (k_a[written] - k_b[written]).abs().max() <= 2.0**-6 * k_a[written].abs().max()
    assert (v_a[written] - v_b[written]).abs().max() <= 2.0**-7 * v_a[written].abs().max()
    # and against the plain formulas
    xq = (x.double() @ w.double().T).view(n_tokens, n_q + 2 * n_kv, d)
    c, s = plain.rotary_tables(torch.tensor(pos), d, theta)
    want_q = plain.apply_rotary(plain.rms_norm(xq[:, :n_q], wq.double(), eps), c.double(), s.double())
    assert (q_b.double() - want_q).abs().max() <= 2.0**-7 * want_q.abs().max() + 1e-3


# ------------------------------------------------------------------ few-token product (weights prefetched into shared memory)
@pytest.mark.parametrize("m,n,k,swiglu,out_dtype", [
    (8, 4096, 1024, False, torch.bfloat16), (8, 6144, 1024, True, torch.bfloat16), (1, 1024, 3072, False, torch.bfloat16),
    (16, 1024, 2048, False, torch.float32), (9, 1000, 200, False, torch.bfloat16), (3, 446, 72, True, torch.bfloat16),
    (5, 77, 8, False, torch.float32), (12, 9472, 64, False, torch.float32), (2, 7, 4104, False, torch.bfloat16),
    (16, 6144, 1024, True, torch.bfloat16), (11, 1176, 520, False, torch.bfloat16),
    # a block's share of the weights exceeds shared memory: several rounds
    (16, 4096, 4104, False, torch.bfloat16), (5, 9472, 520, True, torch.bfloat16), (8, 2048, 8192, False, torch.float32),
    # 17 to 32 tokens: two MMAs' worth of tokens per weight piece, all activations in registers
    (17, 4096, 1024, False, torch.bfloat16), (32, 6144, 1024, True, torch.bfloat16), (25, 1000, 264, False, torch.float32),
    (31, 446, 520, True, torch.bfloat16)])
def test_gemv_against_plain_product(m, n, k, swiglu, out_dtype):
    x = rand(m, k, seed=1).to(torch.bfloat16)
    w = rand(n, k, seed=2, scale=k**-0.5).to(torch.bfloat16)
    got = F().gemv(x.to(DEV), w.to(DEV), out_dtype, swiglu=swiglu)
    y = x.double() @ w.double().T
    if swiglu:
        g, u = y[:, 0::2], y[:, 1::2]
        y = g * torch.sigmoid(g) * u
    assert got.dtype == out_dtype and tuple(got.shape) == tuple(y.shape)
    tol = 2.0**-8 * y.abs().max().item() + 1e-5 if out_dtype == torch.bfloat16 else 1e-5 * max(1.0, y.abs().max().item())
    assert (got.double().cpu() - y).abs().max().item() <= tol


@pytest.mark.parametrize("m,n,k,swiglu,weight_dtype", [(8, 4096, 1024, False, torch.float32), (1, 6144, 1024, True, torch.float32),
                                                        (16, 1000, 520, False, torch.bfloat16), (11, 446, 72, True, torch.float32),
                                                        (3, 2048, 1000, False, torch.bfloat16)])
def test_gemv_with_the_norm_on_load(m, n, k, swiglu, weight_dtype):
    """The few-token product that forms its activations itself as the RMSNorm of a 32-bit stream's rows."""
    eps = 1e-5
    h = rand(m, k, seed=1, scale=3.0).float()
    h[0] *= 40.0  # rows of very different sizes: a scale taken from another row would show
    nw = (1 + 0.1 * rand(k, seed=3)).to(weight_dtype)
    w = rand(n, k, seed=2, scale=k**-0.5).to(torch.bfloat16)
    assert F().gemv_normed_suits(m, n, k, torch.device(DEV))
    got = F().gemv_stream(w.to(DEV), norm=(h.to(DEV), nw.to(DEV), eps), swiglu=swiglu)
    x = plain.rms_norm(h.double(), nw.double(), eps).to(torch.bfloat16).double()  # the product's operand is bfloat16
    y = x @ w.double().T
    if swiglu:
        g, u = y[:, 0::2], y[:, 1::2]
        y = g * torch.sigmoid(g) * u
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == tuple(y.shape)
    # the operand may round the other way where the 32-bit norm lands on the other side of a bfloat16 boundary
    assert (got.double().cpu() - y).abs().max().item() <= 2.0**-7 * y.abs().max().item() + 1e-5
    assert not F().gemv_normed_suits(17, n, k, torch.device(DEV)) and not F().gemv_normed_suits(m, n, 2048, torch.device(DEV))
    with pytest.raises(Exception, match="norm on load"):
        F().gemv_stream(torch.zeros(64, 2048, dtype=torch.bfloat16, device=DEV), norm=(torch.zeros(2, 2048, device=DEV), torch.ones(2048, device=DEV), eps))


@pytest.mark.parametrize("m,n,k", [(8, 1024, 2048), (1, 1024, 3072), (16, 1000, 520), (5, 78, 8), (12, 2560, 4096)])
def test_gemv_adds_into_the_stream(m, n, k):
    """The few-token product whose output stage adds the result, rounded to bfloat16, into a 32-bit stream."""
    x = rand(m, k, seed=1).to(torch.bfloat16)
    w = rand(n, k, seed=2, scale=k**-0.5).to(torch.bfloat16)
    h = rand(m, n, seed=4, scale=5.0).float()
    stream = h.clone().to(DEV)
    assert F().gemv_stream(w.to(DEV), x=x.to(DEV), resid=stream) is None
    y = (x.double() @ w.double().T).to(torch.bfloat16).double()
    want = h.double() + y
    assert (stream.double().cpu() - want).abs().max().item() <= 2.0**-8 * y.abs().max().item() + 1e-5
    # and exactly what the plain product followed by an add gives
    plain_product = F().gemv(x.to(DEV), w.to(DEV), torch.bfloat16)
    assert torch.equal(stream, h.to(DEV) + plain_product.float())
    with pytest.raises(Exception, match="8-byte aligned rows"):  # a stream with rows of an odd number of elements
        F().gemv_stream(w[:77].contiguous().to(DEV), x=x.to(DEV), resid=torch.zeros(m, 77, device=DEV))


def test_gemv_refuses_what_it_cannot_take():
    x = torch.zeros(33, 512, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 512, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="32 tokens"):
        F().gemv(x, w)
    with pytest.raises(Exception, match="17 to 32 tokens"):  # K too long for the activations to stay in registers
        F().gemv(torch.zeros(17, 2048, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 2048, dtype=torch.bfloat16, device=DEV))
    assert not F().gemv_suits(17, 1024, 2048, torch.device(DEV)) and F().gemv_suits(17, 4096, 1024, torch.device(DEV))
    with pytest.raises(Exception, match="weight rows"):
        F().gemv(x[:2], torch.zeros(F().gemv_max_rows(torch.device(DEV)) + 8, 512, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(Exception, match="multiples of 8"):
        F().gemv(torch.zeros(2, 12, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 12, dtype=torch.bfloat16, device=DEV))


# ------------------------------------------------------------------ pairs of blocks on one tile (tcgen05 cta_group::2)
@pytest.fixture
def gemm_pairs_forced():
    before = F().set_gemm_pairs(1)
    yield
    F().set_gemm_pairs(before)


@pytest.mark.parametrize("m,n,k,swiglu", [(2048, 4096, 1024, False), (2048, 6144, 1024, True), (1000, 31000, 200, False),
                                          (4097, 8200, 72, True), (16384, 1024, 64, False)])
def test_gemm_tc_pairs_against_plain_product(gemm_pairs_forced, m, n, k, swiglu):
    x = rand(m, k, seed=1).to(torch.bfloat16)
    w = rand(n, k, seed=2, scale=k**-0.5).to(torch.bfloat16)
    got = F().gemm_tc(x.to(DEV), w.to(DEV), swiglu=swiglu)
    F().check_kernel_errors()
    rows = torch.cat([torch.arange(0, 260), torch.arange(m - 260, m), torch.arange(m // 2, m // 2 + 130)])
    y = x.double()[rows] @ w.double().T
    if swiglu:
        g, u = y[:, 0::2], y[:, 1::2]
        y = g * torch.sigmoid(g) * u
    assert (got.cpu().double()[rows] - y).abs().max().item() <= BF16_ULP * y.abs().max().item() + 1e-4
    # and bit for bit what single blocks on 128 x 256 tiles give (the same products added in the same order)
    F().set_gemm_pairs(0)
    assert torch.equal(got, F().gemm_tc(x.to(DEV), w.to(DEV), swiglu=swiglu))


def test_gemm_tc_qkv_in_pairs_equals_single_blocks():
    n_q, n_kv, d, hidden, dtype = 16, 8, 128, 1024, torch.bfloat16
    lens = [900, 1100]
    n_tokens, width = sum(lens), (n_q + 2 * n_kv) * d
    x = rand(n_tokens, hidden, seed=1).to(dtype).to(DEV)
    w = rand(width, hidden, seed=2, scale=hidden**-0.5).to(dtype).to(DEV)
    wq, wk = (1 + 0.1 * rand(d, seed=3)).float().to(DEV), (1 + 0.1 * rand(d, seed=4)).float().to(DEV)
    cos, sin = plain.rotary_tables(torch.arange(max(lens)), d, 1e5)
    cos, sin = cos[:, : d // 2].contiguous().to(DEV), sin[:, : d // 2].contiguous().to(DEV)
    pos = torch.tensor([p for n in lens for p in range(n)], dtype=torch.int32).to(DEV)
    seq = torch.tensor([i for i, n in enumerate(lens) for _ in range(n)], dtype=torch.int32).to(DEV)
    results = []
    before = F().set_gemm_pairs(0)
    try:
        for mode in (0, 1):
            F().set_gemm_pairs(mode)
            kv, slots, table = scrambled_pages(2, max(lens), n_kv, d, dtype, seed=17)
            q = F().gemm_tc_qkv(x, w, n_q, n_kv, d, wq, wk, 1e-6, cos, sin, pos, seq, slots.to(DEV), kv, max(lens) - 1)
            F().check_kernel_errors()
            results.append((q.clone(), kv.k.clone(), kv.v.clone()))
    finally:
        F().set_gemm_pairs(before)
    for a, b in zip(*results):
        assert torch.equal(torch.nan_to_num(a.float(), nan=-7.0), torch.nan_to_num(b.float(), nan=-7.0))

"""The entry point that allocates nothing: ``gk_attention_decode_bf16_no_alloc``.

Some users of the kernel library cannot allocate device memory while they decode — a server that
has given all free memory to its key/value cache, a C host without PyTorch's allocator, a loop that
cannot afford the device-wide synchronisation of cudaMalloc.  For them the split-KV decode attention
is also exported in a form whose scratch is a fixed array inside the library.  This test calls that
form through its exported C symbol and checks that it gives what the ordinary entry point (scratch
allocated by the caller) gives, twice in a row with different inputs, so that what the first call
leaves in the shared scratch cannot leak into the second.  The file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seed, lens, n_q, n_kv, d):
    from gtar_kimik3_public_b200.ops import functional as F

    gen = torch.Generator().manual_seed(seed)
    n = len(lens)
    per_seq = -(-max(lens) // 64)
    n_pages = n * per_seq + 2
    order = torch.randperm(n_pages, generator=gen)[: n * per_seq].to(torch.int32).view(n, per_seq)
    k = torch.full((n_pages, n_kv, 64, d), float("nan"), dtype=torch.bfloat16)
    v = torch.full((n_pages, n_kv, 64, d), float("nan"), dtype=torch.bfloat16)
    for i, length in enumerate(lens):
        for p in range(-(-length // 64)):
            rows = min(64, length - 64 * p)
            k[order[i, p], :, :rows] = torch.randn(n_kv, rows, d, generator=gen).to(torch.bfloat16)
            v[order[i, p], :, :rows] = torch.randn(n_kv, rows, d, generator=gen).to(torch.bfloat16)
    q = torch.randn(n, n_q, d, generator=gen).to(torch.bfloat16)
    kv = F.PagedKV(k.to(DEV), v.to(DEV), order.contiguous().to(DEV))
    return q.to(DEV), kv, torch.tensor(lens, dtype=torch.int32).to(DEV), torch.arange(n, dtype=torch.int32).to(DEV)


def _call_no_alloc(q, kv, kv_len, slots, scale, n_splits):
    from gtar_kimik3_public_b200.ops import library

    lib = library.library()
    fn = lib.gk_attention_decode_bf16_no_alloc  # the exported C symbol itself
    out = torch.empty_like(q)
    status = fn(q.data_ptr(), kv.k.data_ptr(), kv.v.data_ptr(), out.data_ptr(), kv_len.data_ptr(), slots.data_ptr(),
                kv.block_table.data_ptr(), q.shape[0], q.shape[1], kv.k.shape[1], q.shape[2], kv.max_pages, 64,
                ctypes.c_float(scale), 0, n_splits, torch.cuda.current_stream().cuda_stream)
    return status, out, lib.gk_last_error().decode()


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from gtar_kimik3_public_b200.ops import functional as F

    for seed, lens, n_q, n_kv, d, n_splits in ((1, [700, 64, 1, 333], 16, 8, 128, 5), (2, [100, 900, 65], 4, 1, 64, 7)):
        q, kv, kv_len, slots = _inputs(seed, lens, n_q, n_kv, d)
        want = F.attention_decode(q, kv, kv_len, slots, d**-0.5, 0, n_splits, use_scratch=True)
        torch.cuda.synchronize()
        status, got, message = _call_no_alloc(q, kv, kv_len, slots, d**-0.5, n_splits)
        torch.cuda.synchronize()
        assert status == 0, message
        assert torch.isfinite(got.float()).all()
        # the same kernels on the same inputs: the tolerance of the decode-attention tests holds with room to spare
        scale = want.float().abs().max().item()
        assert (got.float() - want.float()).abs().max().item() <= 2.0**-8 * scale + 2e-3
        assert torch.equal(got, want)  # and in fact the same bits


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    q, kv, kv_len, slots = _inputs(3, [64] * 64, 16, 8, 128)
    status, _, message = _call_no_alloc(q, kv, kv_len, slots, 128**-0.5, 64)  # 64 x 16 x 64 x 130 floats = 34 MB
    assert status != 0 and "scratch" in message and "bytes" in message

"""The cache's bookkeeping: no slot or page lost, held twice or freed twice; windows give pages
back; fixed-size state starts at zero for every new sequence."""

import random

import pytest
import torch

from gtar_kimik3_public_b200.cache import Cache, CacheFull, CacheLayout, PageAllocator, SlotAllocator
from gtar_kimik3_public_b200.parts.base import KVRequest, StateRequest


def test_slot_allocator_reuses_and_refuses_misuse():
    slots = SlotAllocator(3)
    a, b, c = slots.alloc(), slots.alloc(), slots.alloc()
    assert sorted((a, b, c)) == [0, 1, 2]
    with pytest.raises(CacheFull):
        slots.alloc()
    slots.free(b)
    with pytest.raises(ValueError):
        slots.free(b)  # freed twice
    with pytest.raises(ValueError):
        slots.free(7)  # never handed out
    assert slots.alloc() == b  # used again
    assert slots.n_used == 3 and slots.n_free == 0


def test_page_allocator_refuses_misuse():
    pages = PageAllocator(4)
    got = pages.alloc(3)
    assert len(set(got)) == 3
    with pytest.raises(CacheFull):
        pages.alloc(2)
    assert pages.n_used == 3  # a refused request takes nothing
    pages.free(got[:2])
    with pytest.raises(ValueError):
        pages.free([got[0]])
    with pytest.raises(ValueError):
        pages.free([got[2], got[2]])
    assert pages.n_used == 1


def _layout():
    full = KVRequest(2, 16)
    window = KVRequest(2, 16, window=100)
    state = StateRequest((4, 3))
    return CacheLayout([full, window, full, state, None, full], shared_with={5: 0})


def test_groups_have_storage_of_their_own():
    cache = Cache(_layout(), max_tokens=64 * 20, dtype=torch.float32, device="cpu", max_seqs=4)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 1
    full, window = cache.kv_groups
    assert full.entries == [0, 2] and window.entries == [1]
    assert full.k.shape == (2, 20, 2, 64, 16)
    assert window.k.shape[1] == 20 and window.k.data_ptr() != full.k.data_ptr()
    assert cache.view(4) is None
    assert cache.view(5).k.data_ptr() == cache.view(0).k.data_ptr()  # entry 5 reads entry 0's storage
    assert cache.is_shared(5) and not cache.is_shared(0)
    assert cache.view(2).k.data_ptr() != cache.view(0).k.data_ptr()
    assert cache.view(3).shape == (4, 4, 3)


def test_random_traffic_keeps_the_invariants():
    rng = random.Random(0)
    cache = Cache(_layout(), max_tokens=64 * 24, dtype=torch.float32, device="cpu", max_seqs=5, max_seq_len=640)
    live = {}
    before = {}
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and cache.slots.n_free:
            live[cache.open()] = 0
        elif action < 0.45 and live:
            slot = rng.choice(list(live))
            cache.close(slot)
            del live[slot]
        elif live:
            slot = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 7, 64, 130])
            if cache.can_grow({slot: n}):
                assert cache.grow(slot, n) == live[slot]
                before[slot] = live[slot]
                live[slot] += n
            else:
                with pytest.raises(CacheFull):
                    cache.grow(slot, n)
                    raise CacheFull("fits the pages but not checked")  # pragma: no cover
        cache.sync()
        cache.check_invariants()
        full, window = cache.kv_groups
        for slot, length in live.items():
            assert cache.length[slot] == length
            assert len(full.owned[slot]) == -(-length // 64)
            if length:  # the window group holds the pages its last step could read, no more
                first = max(0, before[slot] - 100 + 1) // 64
                assert sorted(window.owned[slot]) == list(range(first, (length - 1) // 64 + 1))
            for index, page in full.owned[slot].items():
                assert full.table[slot, index] == page
    for slot in list(live):
        cache.close(slot)
    cache.check_invariants()
    assert all(g.pages.n_used == 0 for g in cache.kv_groups) and cache.slots.n_used == 0


def test_window_pages_go_back_to_the_pool():
    cache = Cache(CacheLayout([KVRequest(1, 16, window=64)]), max_tokens=64 * 8, dtype=torch.float32, device="cpu", max_seqs=1)
    slot = cache.open()
    group = cache.kv_groups[0]
    for _ in range(500):
        cache.grow(slot, 1)
        assert group.pages.n_used <= 2
    assert sorted(group.owned[slot]) == [6, 7]


def test_state_is_zero_for_every_new_sequence():
    cache = Cache(CacheLayout([StateRequest((3,))]), max_tokens=64, dtype=torch.float32, device="cpu", max_seqs=1)
    slot = cache.open()
    cache.view(0)[slot] += 5.0
    cache.close(slot)
    again = cache.open()
    assert again == slot and torch.all(cache.view(0)[again] == 0)


def test_limits():
    cache = Cache(CacheLayout([KVRequest(1, 16)]), max_tokens=200, dtype=torch.float32, device="cpu", max_seq_len=130)
    assert cache.n_pages == 4 and cache.max_seq_len == 130
    a, b = cache.open(), cache.open()
    cache.grow(a, 129)
    with pytest.raises(CacheFull):
        cache.grow(a, 2)  # beyond the longest sequence
    assert cache.can_grow({b: 64}) and not cache.can_grow({b: 65})
    with pytest.raises(CacheFull):
        cache.grow(b, 65)
    cache.check_invariants()
    with pytest.raises(ValueError):
        Cache(CacheLayout([None, KVRequest(1, 16)], shared_with={1: 0}), 64, torch.float32, "cpu")

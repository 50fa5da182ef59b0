"""The cache: a slot for each live sequence; keys and values in pages; per-sequence state.

The reference keeps, per layer, dense ``[batch, kv_heads, max_seq_len, head_dim]`` buffers and one
length for the whole batch (src/cache.py:4-17), and for its other architecture a state of
fixed size per batch row (src/cache.py:48-57).  Here

* a *slot* stands for one sequence: it has its own length, a row of every group's page table
  and a row of every state tensor; slots are given back when a sequence ends and used again;
* keys and values live in *pages* of ``page_size`` positions, ``[page, kv_head, page_size,
  head_dim]`` per layer, handed to a sequence as it grows, so the pool is sized by the tokens that
  live sequences hold (each rounded up to a page) and not by slots times the longest context;
* layers whose mixers ask for the same kind of storage form a *group* with tensors and a page
  pool of its own: one group for "all positions", one per window length (pages that have left
  the window go back to the pool), one per shape of fixed-size state;
* stale data is never cleared from pages: nothing reads beyond a sequence's length (the
  reference argues the same for its rollback, src/cache.py:37-45).  State rows are zeroed when
  a slot is handed out.

Which entry of the model's run list uses which storage is given by ``CacheLayout``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..ops.functional import DecodeWork, PagedKV
from ..parts.base import KVRequest, StateRequest
from .allocators import CacheFull, PageAllocator, SlotAllocator

PAGE_SIZE = 64


def rounded_tokens(n_tokens: int, page_size: int = PAGE_SIZE) -> int:
    """What a sequence of ``n_tokens`` counts against a cache's ``max_tokens``: its length rounded up to whole pages."""
    return -(-int(n_tokens) // page_size) * page_size


@dataclass
class CacheLayout:
    """``requests[e]`` is what entry ``e`` of the model's run list needs kept: one request, None, or a
    list of requests (keys and values and a state, several states of their own shapes and types: the
    reference's fixed-size example holds a 32-bit matrix and three rolling buffers, src/cache.py:48-57).
    An entry may instead read the storage of an earlier entry: ``shared_with[e] = e'``."""

    requests: list[KVRequest | StateRequest | None | list | tuple]
    shared_with: dict[int, int] = field(default_factory=dict)

    def items_of(self, entry: int) -> tuple:
        """The entry's requests as a tuple (empty for None)."""
        request = self.requests[entry]
        if request is None:
            return ()
        return tuple(request) if isinstance(request, (list, tuple)) else (request,)


class _KVGroup:
    def __init__(self, request: KVRequest, items: list[tuple[int, int]], n_slots: int, n_pages: int, max_pages_per_seq: int,
                 page_size: int, dtype: torch.dtype, device: torch.device):
        # items: (run-list entry, place among that entry's requests) of everything stored here
        self.request, self.items, self.page_size = request, items, page_size
        self.entries = [entry for entry, _ in items]
        self.index_of = {item: i for i, item in enumerate(items)}
        shape = (len(items), n_pages, request.n_kv_heads, page_size, request.head_dim)
        self.k = torch.empty(shape, dtype=dtype, device=device)
        self.v = torch.empty(shape, dtype=dtype, device=device)
        self.pages = PageAllocator(n_pages)
        self.max_pages_per_seq = max_pages_per_seq
        self.table_host = np.zeros((n_slots, max_pages_per_seq), dtype=np.int32)
        self.table = torch.zeros((n_slots, max_pages_per_seq), dtype=torch.int32, device=device)
        self.owned: dict[int, dict[int, int]] = {}  # slot -> {page index in sequence: page}
        self.upto: dict[int, int] = {}  # slot -> one past the highest page index the sequence ever had
        self.dirty: set[int] = set()
        self._staging = None  # pinned copies of the table for uploads, made at the first upload
        self._work = None  # decode attention's scratch for this group's layers, made with the first view

    def open_slot(self, slot: int) -> None:
        self.owned[slot] = {}
        self.upto[slot] = 0

    def close_slot(self, slot: int) -> None:
        self.pages.free(self.owned.pop(slot).values())
        del self.upto[slot]

    def pages_needed(self, slot: int, old_len: int, new_len: int) -> int:
        # a sequence only grows, so the pages it lacks are those from `upto` on (a window may have skipped some)
        first, last = self._span(old_len, new_len)
        return max(0, last + 1 - max(first, self.upto[slot]))

    def _span(self, old_len: int, new_len: int) -> tuple[int, int]:
        """Page indices that hold positions a step from old_len to new_len reads or writes."""
        first = 0
        if self.request.window is not None:
            first = max(0, old_len - self.request.window + 1) // self.page_size
        return first, (new_len - 1) // self.page_size

    def grow(self, slot: int, old_len: int, new_len: int) -> None:
        if new_len <= 0:
            return
        first, last = self._span(old_len, new_len)
        if last >= self.max_pages_per_seq:
            raise CacheFull(f"a sequence of {new_len} tokens exceeds the longest the cache was sized for "
                            f"({self.max_pages_per_seq * self.page_size})")
        owned = self.owned[slot]
        if self.request.window is not None:  # pages wholly before the window go back to the pool
            gone = [i for i in owned if i < first]
            if gone:
                self.pages.free([owned.pop(i) for i in gone])
        begin = max(first, self.upto[slot])
        if begin <= last:
            missing = list(range(begin, last + 1))
            pages = self.pages.alloc(len(missing))
            owned.update(zip(missing, pages))
            self.table_host[slot, begin:last + 1] = pages
            self.upto[slot] = last + 1
            self.dirty.add(slot)

    STAGING_RING = 8

    def sync(self) -> None:
        """Sends the changed rows of the page table to the device.  The rows are copied into a
        pinned buffer of their own first: the host goes on changing ``table_host`` (a slot that is
        given back and used again) while earlier copies may still wait in the stream, and a copy
        must carry the numbers of the step it was issued for.  The pinned buffers are a small ring,
        each guarded by an event, so that none is written while a copy out of it may still wait."""
        if not self.dirty:
            return
        slots = sorted(self.dirty)
        if not self.table.is_cuda:
            self.table[slots] = torch.from_numpy(self.table_host[slots])
            self.dirty.clear()
            return
        if self._staging is None:
            self._staging = [torch.empty(self.table_host.shape, dtype=torch.int32).pin_memory() for _ in range(self.STAGING_RING)]
            self._staging_np = [t.numpy() for t in self._staging]
            self._staging_events = [None] * self.STAGING_RING
            self._staging_turn = 0
        turn = self._staging_turn
        self._staging_turn = (turn + 1) % self.STAGING_RING
        if self._staging_events[turn] is not None:
            self._staging_events[turn].synchronize()
        staged, staged_np = self._staging[turn], self._staging_np[turn]
        for slot in slots:
            staged_np[slot] = self.table_host[slot]
            self.table[slot].copy_(staged[slot], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._staging_events[turn] = event
        self.dirty.clear()

    def view(self, item: tuple[int, int]) -> PagedKV:
        i = self.index_of[item]
        if self._work is None and self.table.is_cuda:
            self._work = DecodeWork(self.table.device)
        return PagedKV(self.k[i], self.v[i], self.table, self._work)


class _StateGroup:
    def __init__(self, request: StateRequest, items: list[tuple[int, int]], n_slots: int, device: torch.device):
        self.request, self.items = request, items
        self.entries = [entry for entry, _ in items]
        self.index_of = {item: i for i, item in enumerate(items)}
        self.state = torch.zeros((len(items), n_slots, *request.shape), dtype=request.dtype, device=device)

    def open_slot(self, slot: int) -> None:
        self.state[:, slot].zero_()

    def view(self, item: tuple[int, int]) -> torch.Tensor:
        return self.state[self.index_of[item]]


class Cache:
    """Storage for up to ``max_seqs`` live sequences holding at most ``max_tokens`` tokens in all,
    each sequence's count rounded up to a multiple of the page size."""

    def __init__(self, layout: CacheLayout, max_tokens: int, dtype: torch.dtype, device: torch.device | str,
                 max_seqs: int | None = None, max_seq_len: int | None = None, page_size: int = PAGE_SIZE):
        device = torch.device(device)
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if page_size % 32:
            raise ValueError("page_size must be a multiple of 32")
        self.layout, self.dtype, self.device, self.page_size = layout, dtype, device, page_size
        self.n_pages = -(-max_tokens // page_size)
        self.max_seqs = min(self.n_pages, max_seqs if max_seqs else 256)
        pages_per_seq = self.n_pages if max_seq_len is None else min(self.n_pages, -(-max_seq_len // page_size))
        self.max_seq_len = pages_per_seq * page_size if max_seq_len is None else min(max_seq_len, pages_per_seq * page_size)
        self.slots = SlotAllocator(self.max_seqs)
        self.length: dict[int, int] = {}
        self.kv_groups: list[_KVGroup] = []
        self.state_groups: list[_StateGroup] = []
        self._where: dict[tuple[int, int], object] = {}
        by_request: dict[object, list[tuple[int, int]]] = {}
        for entry in range(len(layout.requests)):
            if entry in layout.shared_with:
                continue
            for place, request in enumerate(layout.items_of(entry)):
                by_request.setdefault(request, []).append((entry, place))
        for request, entries in by_request.items():
            if isinstance(request, KVRequest):
                # A windowed group draws on a pool as large as the others': a long prompt needs all its
                # pages while its step runs.  What the window saves is returned at the sequence's
                # next step, so fewer pages are *in use*, and more sequences fit, than without it.
                n_pages = self.n_pages
                group = _KVGroup(request, entries, self.max_seqs, n_pages, pages_per_seq, page_size, dtype, device)
                self.kv_groups.append(group)
            elif isinstance(request, StateRequest):
                group = _StateGroup(request, entries, self.max_seqs, device)
                self.state_groups.append(group)
            else:
                raise TypeError(f"unknown cache request {request!r}")
            for item in entries:
                self._where[item] = group
        for entry, source in layout.shared_with.items():
            if not layout.items_of(source) or source in layout.shared_with:
                raise ValueError(f"run-list entry {entry} shares the cache of entry {source}, which keeps nothing of its own")

    # ------------------------------------------------------------------ slots
    def open(self) -> int:
        """A slot for a new sequence: length 0, no pages, zero state."""
        slot = self.slots.alloc()
        self.length[slot] = 0
        for group in self.kv_groups:
            group.open_slot(slot)
        for group in self.state_groups:
            group.open_slot(slot)
        return slot

    def close(self, slot: int) -> None:
        """Gives back the slot and everything the sequence holds."""
        self.slots.free(slot)
        del self.length[slot]
        for group in self.kv_groups:
            group.close_slot(slot)

    def can_grow(self, growth: dict[int, int]) -> bool:
        """Whether ``growth[slot]`` more tokens for each listed slot fit in the free pages."""
        for group in self.kv_groups:
            need = sum(group.pages_needed(s, self.length[s], self.length[s] + n) for s, n in growth.items() if n > 0)
            if need > group.pages.n_free:
                return False
        return all(self.length[s] + n <= self.max_seq_len for s, n in growth.items())

    def grow(self, slot: int, n_new: int) -> int:
        """Makes room for ``n_new`` more tokens of the sequence in ``slot`` and counts them in.
        Returns the length before."""
        if not self.slots.in_use(slot):
            raise ValueError(f"slot {slot} is not in use")
        old = self.length[slot]
        new = old + n_new
        if new > self.max_seq_len:
            raise CacheFull(f"sequence would reach {new} tokens; the cache holds sequences up to {self.max_seq_len}")
        for group in self.kv_groups:
            group.grow(slot, old, new)
        self.length[slot] = new
        return old

    def sync(self) -> None:
        """Brings the device page tables up to date; call after ``grow`` and before the step runs."""
        for group in self.kv_groups:
            group.sync()

    # ------------------------------------------------------------------ views
    def view(self, entry: int):
        """Storage of run-list entry ``entry``: a ``PagedKV`` or a state tensor ``[n_slots, ...]`` for a single
        request, None for none, and for a list of requests a tuple of those in the list's order."""
        source = self.layout.shared_with.get(entry, entry)
        request = self.layout.requests[source]
        if request is None:
            return None
        views = tuple(self._where[(source, place)].view((source, place)) for place in range(len(self.layout.items_of(source))))
        return views if isinstance(request, (list, tuple)) else views[0]

    def is_shared(self, entry: int) -> bool:
        return entry in self.layout.shared_with

    # ------------------------------------------------------------------ accounting
    def live_tokens(self) -> int:
        return sum(self.length.values())

    def kv_bytes_per_token(self) -> int:
        total = 0
        for group in self.kv_groups:
            r = group.request
            total += 2 * len(group.items) * r.n_kv_heads * r.head_dim * self.k_element_size()
        return total

    def k_element_size(self) -> int:
        return torch.empty((), dtype=self.dtype).element_size()

    def check_invariants(self) -> None:
        """No page held twice, none lost, lengths only for slots in use."""
        for group in self.kv_groups:
            held = [p for owned in group.owned.values() for p in owned.values()]
            assert len(held) == len(set(held)), "a page is held by two sequences"
            assert len(held) == group.pages.n_used, "pages were lost"
            assert set(group.owned) == set(self.length), "a group tracks other slots than the cache"
        assert len(self.length) == self.slots.n_used

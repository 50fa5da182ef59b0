"""Host-side bookkeeping of the cache: which slots and which pages are in use.

Both allocators refuse misuse loudly (a slot or page freed twice, one never handed out, more
asked than there is) because a silent mistake here shows up much later as one sequence reading
another's keys.
"""

from __future__ import annotations


class CacheFull(RuntimeError):
    """No free slot or not enough free pages for what was asked."""


class SlotAllocator:
    """Slots ``0..n-1``; a freed slot is handed out again (lowest number first)."""

    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise ValueError("a cache needs at least one slot")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))  # pop() gives the lowest
        self._used: set[int] = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} slots are in use")
        slot = self._free.pop()
        self._used.add(slot)
        return slot

    def free(self, slot: int) -> None:
        if slot not in self._used:
            raise ValueError(f"slot {slot} is not in use (freed twice, or never handed out)")
        self._used.remove(slot)
        self._free.append(slot)
        self._free.sort(reverse=True)

    @property
    def n_used(self) -> int:
        return len(self._used)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def in_use(self, slot: int) -> bool:
        return slot in self._used


class PageAllocator:
    """Pages ``0..n-1`` of a pool, handed out one by one."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._used: set[int] = set()

    def alloc(self, count: int = 1) -> list[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} pages asked, {len(self._free)} of {self.n_pages} free")
        pages = [self._free.pop() for _ in range(count)]
        self._used.update(pages)
        return pages

    def free(self, pages) -> None:
        pages = list(pages)
        for page in pages:
            if page not in self._used:
                raise ValueError(f"page {page} is not in use (freed twice, or never handed out)")
        if len(set(pages)) != len(pages):
            raise ValueError("a page is listed twice in one free")
        for page in pages:
            self._used.remove(page)
            self._free.append(page)

    @property
    def n_used(self) -> int:
        return len(self._used)

    @property
    def n_free(self) -> int:
        return len(self._free)

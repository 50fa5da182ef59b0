"""Slots, pages and per-sequence state."""

from .allocators import CacheFull, PageAllocator, SlotAllocator  # noqa: F401
from .cache import PAGE_SIZE, Cache, CacheLayout, rounded_tokens  # noqa: F401

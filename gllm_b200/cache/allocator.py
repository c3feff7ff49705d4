"""Page and slot allocators (host side, no device work).

The reference keeps a free list, an "active" dict with reference counts and a
"cached" dict that released pages move to and can never leave
(gllm/model/kv_cache/paged_kv_cache.py:47-57,81-110): once the free list is
empty, reserving raises although released pages exist.  Here a released page
goes straight back to the free list and is handed out again; taking a page
twice, freeing one twice or freeing a page nobody holds raises.
"""

from __future__ import annotations


class CacheError(RuntimeError):
    """The cache manager was asked for something inconsistent."""


class OutOfPages(CacheError):
    """Not enough free pages (or slots); nothing was taken."""

    def __init__(self, needed: int, free: int, what: str = "pages"):
        super().__init__(f"{needed} {what} needed, {free} free")
        self.needed = needed
        self.free = free


class BlockAllocator:
    """Fixed pool of ``num_blocks`` pages with ids ``0 .. num_blocks-1``."""

    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        self.num_blocks = int(num_blocks)
        # LIFO: the page freed last is handed out first, so reuse happens early.
        self._free = list(range(self.num_blocks - 1, -1, -1))
        self._held = bytearray(self.num_blocks)
        self.total_allocated = 0
        self.total_reused = 0
        self._ever_used = bytearray(self.num_blocks)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_blocks - len(self._free)

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self, n: int) -> list[int]:
        """Take ``n`` pages, or raise OutOfPages and take none."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(n, len(self._free))
        out = []
        for _ in range(n):
            b = self._free.pop()
            if self._held[b]:
                raise CacheError(f"page {b} was on the free list while held")
            self._held[b] = 1
            if self._ever_used[b]:
                self.total_reused += 1
            self._ever_used[b] = 1
            out.append(b)
        self.total_allocated += n
        return out

    def free(self, blocks) -> None:
        blocks = list(blocks)
        for b in blocks:
            if not 0 <= b < self.num_blocks:
                raise CacheError(f"page {b} is outside the pool of {self.num_blocks}")
            if not self._held[b]:
                raise CacheError(f"page {b} is freed but nobody holds it")
        if len(set(blocks)) != len(blocks):
            raise CacheError("a page is freed twice in one call")
        for b in blocks:
            self._held[b] = 0
            self._free.append(b)

    def is_held(self, block: int) -> bool:
        return bool(self._held[block])


class SlotAllocator:
    """State slots ``0 .. n-1``: one per live request, never moved.

    The reference's per-request row index is compacted every step by copying
    rows (gllm/llm/llm.py:185-191), which is where its stale ``num_blocks``
    read comes from (gllm/llm/llm.py:176).  A slot here stays put from
    admission to finish.
    """

    def __init__(self, n: int):
        self.n = int(n)
        self._free = list(range(self.n - 1, -1, -1))
        self._held = bytearray(self.n)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages(1, 0, "state slots")
        s = self._free.pop()
        self._held[s] = 1
        return s

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.n or not self._held[slot]:
            raise CacheError(f"state slot {slot} is freed but not held")
        self._held[slot] = 0
        self._free.append(slot)

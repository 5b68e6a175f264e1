"""Page pools: which pages of a cache group are free, and who holds the others.

The free list is a stack (last freed, first taken), as the reference's allocator
(src/wllm/engine/kv_cache.py:27-54), so a page that a finished request gives back
is the next one handed out.  Unlike the reference, exhaustion is a typed exception
and giving back a page that is not held is an error instead of a silent clamp.
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """A cache group has fewer free pages than a step needs."""

    def __init__(self, group: str, needed: int, free: int):
        super().__init__(f"cache group '{group}': {needed} pages needed, {free} free")
        self.group, self.needed, self.free = group, needed, free


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # page 0 is taken first
        self._held = [False] * num_pages
        self.takes = 0   # pages handed out so far; above num_pages means pages were used again

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("?", 1, 0)
        page = self._free.pop()
        self._held[page] = True
        self.takes += 1
        return page

    def give(self, page: int) -> None:
        if not (0 <= page < self.num_pages) or not self._held[page]:
            raise RuntimeError(f"page {page} given back but not held (freed twice?)")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]

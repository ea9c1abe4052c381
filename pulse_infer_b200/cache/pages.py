"""Page accounting on the host: a free list of page ids and the block table of every request slot.

Reference parity: ``src/runtime/block_manager.cpp:8-13,29-31,52-55,93-96`` (LIFO free list whose first
allocation pops the highest id, freed ids are handed out again first), ``block_manager.cpp:61-91``
(invalid id and double free are detected with an allocated-bitmap), ``block_manager.cpp:44-46``
("Insufficient free blocks"), ``src/runtime/block_table.cpp:94-148`` (rows padded with -1).
"""
from __future__ import annotations

import numpy as np


class OutOfPages(RuntimeError):
    """Not enough free pages; nothing was allocated."""


class PageError(RuntimeError):
    """A page id that does not exist, is not allocated, or is freed twice."""


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("num_pages must be positive")
        self.num_pages = num_pages
        self._free = list(range(num_pages))          # pop() takes from the end
        self._allocated = np.zeros(num_pages, dtype=bool)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_allocated(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, count: int) -> list[int]:
        if count < 0:
            raise ValueError("count must not be negative")
        if count > len(self._free):
            raise OutOfPages(f"Insufficient free blocks: want {count}, have {len(self._free)}")
        pages = [self._free.pop() for _ in range(count)]
        for p in pages:
            self._allocated[p] = True
        return pages

    def free(self, pages) -> None:
        pages = list(pages)
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise PageError(f"page id {p} does not exist (pool has {self.num_pages})")
            if not self._allocated[p]:
                raise PageError(f"page {p} is not allocated (double free?)")
        if len(set(pages)) != len(pages):
            raise PageError("a page id appears twice in one free")
        for p in pages:
            self._allocated[p] = False
            self._free.append(p)

    def is_allocated(self, page: int) -> bool:
        return bool(self._allocated[page])


class BlockTable:
    """``table[slot, i]`` = page holding positions ``[i * page_size, (i + 1) * page_size)`` of the
    request in ``slot``, or -1.  Rows changed since the last upload are remembered."""

    def __init__(self, max_slots: int, max_pages_per_request: int):
        self.table = np.full((max_slots, max_pages_per_request), -1, dtype=np.int32)
        self.dirty: set[int] = set()

    def set(self, slot: int, index: int, page: int) -> None:
        self.table[slot, index] = page
        self.dirty.add(slot)

    def clear_row(self, slot: int) -> None:
        self.table[slot, :] = -1
        self.dirty.add(slot)

    def row(self, slot: int) -> np.ndarray:
        return self.table[slot]

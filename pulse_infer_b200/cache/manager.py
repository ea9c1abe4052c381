"""The cache manager: token pages in groups, block tables per request, and fixed-size state slots.

* A **group** collects the caches (one per layer that writes keys and values) whose needs are the
  same: number of kv heads, head size and window.  A group has its own page pool
  ``[caches, 2 (K, V), pages, kv heads, page size, head size]``, its own free list and its own block
  table; one page id addresses the same slot in every cache of the group.  A group with a window
  gives a page back as soon as every position in it has fallen out of the window.
* A request occupies a **slot**: a row of every group's block table plus one entry in every
  per-request state tensor (``[slots, *shape]``, zeroed when the slot is opened) - this is where a
  mixer with recurrent state keeps it.  Qwen3 has none, but the slots exist for any mixer that asks.
* Pages are reserved for a step *before* it runs (``reserve``), lengths are advanced after it
  (``commit``), everything is given back by ``close``.

Reference parity: ``src/runtime/kv_cache_manager.cpp:56-76`` (pools ``[pages, kv heads, page size,
head size]`` per layer for K and for V), ``kv_cache_manager.cpp:83-131`` (allocate / extend by whole
pages), ``kv_cache_manager.cpp:175-196`` (free_sequence returns every page), ``234-253`` (length
bookkeeping).  Unlike the reference, which allocates lazily inside the forward pass
(``src/model/qwen3/model.cpp:1218-1249``) and so can fail half-way, reservation here is atomic.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import CacheSpec, StateSpec
from .pages import BlockTable, OutOfPages, PageAllocator, PageError


class CacheError(RuntimeError):
    pass


@dataclass
class PageGroup:
    spec: CacheSpec
    cache_indices: list            # which of the model's caches live in this group
    allocator: PageAllocator
    table: BlockTable
    pool: torch.Tensor | None = None          # [caches, 2, pages, nkv, page_size, d]
    device_table: torch.Tensor | None = None  # int32 [slots, max_pages]
    first_live: dict = field(default_factory=dict)   # slot -> index of the first page still held

    def kv(self, cache_index: int):
        """Key and value pools of one cache: two tensors [pages, nkv, page_size, d]."""
        local = self.cache_indices.index(cache_index)
        return self.pool[local, 0], self.pool[local, 1]


class CacheManager:
    def __init__(self, cache_specs: list, state_specs: list, page_size: int, num_pages: int, max_slots: int,
                 max_tokens_per_request: int, dtype: torch.dtype = torch.bfloat16, device=None,
                 allocate_pools: bool = True):
        """``cache_specs[i]`` is the CacheSpec of the model's cache i (or None); ``state_specs[j]`` is the
        StateSpec of layer j (or None).  ``num_pages`` is the size of every group's pool."""
        if page_size <= 0 or max_slots <= 0 or max_tokens_per_request <= 0:
            raise ValueError("page_size, max_slots and max_tokens_per_request must be positive")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_slots = max_slots
        self.max_pages_per_request = (max_tokens_per_request + page_size - 1) // page_size
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.groups: list[PageGroup] = []
        self.group_of_cache: dict[int, int] = {}
        by_spec: dict[CacheSpec, int] = {}
        for index, spec in enumerate(cache_specs):
            if spec is None:
                continue
            if spec not in by_spec:
                by_spec[spec] = len(self.groups)
                self.groups.append(PageGroup(spec, [], PageAllocator(num_pages),
                                             BlockTable(max_slots, self.max_pages_per_request)))
            gid = by_spec[spec]
            self.groups[gid].cache_indices.append(index)
            self.group_of_cache[index] = gid
        for g in self.groups:
            g.device_table = torch.full((max_slots, self.max_pages_per_request), -1, dtype=torch.int32,
                                        device=self.device)
            if allocate_pools:
                g.pool = torch.zeros((len(g.cache_indices), 2, num_pages, g.spec.num_kv_heads, page_size,
                                      g.spec.head_dim), dtype=dtype, device=self.device)
        # fixed-size per-request state, one tensor per layer that asks for it
        self.state: dict[int, torch.Tensor] = {}
        for layer, spec in enumerate(state_specs):
            if spec is not None:
                self.state[layer] = torch.zeros((max_slots,) + tuple(spec.shape), dtype=spec.dtype, device=self.device)
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._slot_of: dict = {}            # request id -> slot
        self._length = np.zeros(max_slots, dtype=np.int64)     # committed tokens per slot
        self._reserved = np.zeros(max_slots, dtype=np.int64)   # tokens that pages are reserved for

    # ---- slots -----------------------------------------------------------------------------------
    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def has(self, request_id) -> bool:
        return request_id in self._slot_of

    def slot(self, request_id) -> int:
        if request_id not in self._slot_of:
            raise CacheError(f"request '{request_id}' holds no slot")
        return self._slot_of[request_id]

    def length(self, request_id) -> int:
        return int(self._length[self.slot(request_id)])

    def open(self, request_id) -> int:
        """Give a request a slot: empty block-table rows and zeroed state."""
        if request_id in self._slot_of:
            raise CacheError(f"request '{request_id}' already holds a slot")  # kv_cache_manager.cpp:88-90
        if not self._free_slots:
            raise CacheError("no free request slot")
        slot = self._free_slots.pop()
        self._slot_of[request_id] = slot
        self._length[slot] = 0
        self._reserved[slot] = 0
        for g in self.groups:
            g.table.clear_row(slot)
            g.first_live[slot] = 0
        for tensor in self.state.values():
            tensor[slot].zero_()
        return slot

    # ---- pages -----------------------------------------------------------------------------------
    def _first_needed_page(self, group: PageGroup, length: int) -> int:
        """Pages before this index hold only positions no later query can see."""
        w = group.spec.window
        if w is None:
            return 0
        # a query at position >= length sees keys >= length - w + 1; positions <= length - w are dead
        return max(0, (length - w + 1) // self.page_size)

    def pages_needed(self, request_id, new_length: int) -> list[int]:
        """Per group: how many new pages a reservation up to ``new_length`` tokens would take."""
        slot = self.slot(request_id)
        have = (int(self._reserved[slot]) + self.page_size - 1) // self.page_size
        want = (new_length + self.page_size - 1) // self.page_size
        return [max(0, want - have) for _ in self.groups]

    def pages_for_new_request(self, num_tokens: int) -> list[int]:
        want = (num_tokens + self.page_size - 1) // self.page_size
        return [want for _ in self.groups]

    def free_pages(self) -> list[int]:
        return [g.allocator.num_free for g in self.groups]

    def _covered(self, slot: int, new_length: int) -> bool:
        """True when the pages already reserved for the slot reach new_length (the common decode case)."""
        page = self.page_size
        return new_length <= (int(self._reserved[slot]) + page - 1) // page * page

    def can_reserve(self, request_id, new_length: int) -> bool:
        if self._covered(self.slot(request_id), new_length):
            return new_length <= self.max_pages_per_request * self.page_size
        return all(n <= g.allocator.num_free for n, g in zip(self.pages_needed(request_id, new_length), self.groups))

    def reserve(self, request_id, new_length: int) -> None:
        """Make sure every group holds pages for positions < new_length.  Atomic: on OutOfPages
        nothing has changed."""
        slot = self.slot(request_id)
        if self._covered(slot, new_length) and new_length <= self.max_pages_per_request * self.page_size:
            if new_length > self._reserved[slot]:
                self._reserved[slot] = new_length
            return
        if new_length > self.max_pages_per_request * self.page_size:
            raise CacheError(f"request '{request_id}' would reach {new_length} tokens, beyond the "
                             f"{self.max_pages_per_request * self.page_size} this cache was sized for")
        needed = self.pages_needed(request_id, new_length)
        for n, g in zip(needed, self.groups):
            if n > g.allocator.num_free:
                raise OutOfPages(f"Insufficient free blocks: request '{request_id}' needs {n} more pages, "
                                 f"{g.allocator.num_free} are free")
        have = (int(self._reserved[slot]) + self.page_size - 1) // self.page_size
        for n, g in zip(needed, self.groups):
            for i, page in enumerate(g.allocator.allocate(n)):
                g.table.set(slot, have + i, page)
        self._reserved[slot] = max(int(self._reserved[slot]), new_length)

    def commit(self, request_id, new_length: int) -> None:
        """The step has run: the request now holds ``new_length`` tokens.  Pages that a window has
        passed are given back."""
        slot = self.slot(request_id)
        if new_length > self._reserved[slot]:
            raise CacheError(f"commit of {new_length} tokens beyond the {int(self._reserved[slot])} reserved")
        if new_length < self._length[slot]:
            raise CacheError("a request's length cannot shrink")
        self._length[slot] = new_length
        for g in self.groups:
            first = self._first_needed_page(g, new_length)
            start = g.first_live[slot]
            if first > start:
                dead = [int(g.table.table[slot, i]) for i in range(start, first) if g.table.table[slot, i] >= 0]
                g.allocator.free(dead)
                for i in range(start, first):
                    g.table.set(slot, i, -1)
                g.first_live[slot] = first

    def close(self, request_id) -> None:
        """The request is finished (or preempted): all its pages and its slot are given back."""
        slot = self.slot(request_id)
        for g in self.groups:
            row = g.table.row(slot)
            held = [int(p) for p in row if p >= 0]
            g.allocator.free(held)
            g.table.clear_row(slot)
            g.first_live.pop(slot, None)
        self._length[slot] = 0
        self._reserved[slot] = 0
        del self._slot_of[request_id]
        self._free_slots.append(slot)

    def reset(self) -> None:
        for rid in list(self._slot_of):
            self.close(rid)

    # ---- device side -----------------------------------------------------------------------------
    def sync_tables(self) -> None:
        """Upload the block-table rows that changed since the last call."""
        for g in self.groups:
            if not g.table.dirty:
                continue
            rows = sorted(g.table.dirty)
            host = torch.from_numpy(g.table.table[rows])
            index = torch.tensor(rows, dtype=torch.long)
            if self.device.type == "cuda":
                g.device_table.index_copy_(0, index.to(self.device, non_blocking=True),
                                           host.to(self.device, non_blocking=True))
            else:
                g.device_table.index_copy_(0, index, host)
            g.table.dirty.clear()

    def group_for_cache(self, cache_index: int) -> PageGroup:
        return self.groups[self.group_of_cache[cache_index]]

    # ---- invariants (used by tests) -----------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, none held twice: per group, free + held == pool and held ids are distinct."""
        for g in self.groups:
            held = [int(p) for slot in self._slot_of.values() for p in g.table.row(slot) if p >= 0]
            if len(held) != len(set(held)):
                raise PageError("a page is held by two table entries")
            if len(held) + g.allocator.num_free != g.allocator.num_pages:
                raise PageError(f"pages lost: {len(held)} held + {g.allocator.num_free} free != {g.allocator.num_pages}")
            for p in held:
                if not g.allocator.is_allocated(p):
                    raise PageError(f"page {p} is in a table but marked free")
            for slot in set(range(self.max_slots)) - set(self._slot_of.values()):
                if (g.table.row(slot) >= 0).any():
                    raise PageError(f"free slot {slot} still has pages in its row")

"""The cache of the model's mixers: a slot for each live sequence, keys and values for each cache entry in pages,
fixed-size state beside them.

A *cache entry* is what one run of a layer writes (most models: one per layer). Entries with the same need (kind,
kv heads, head size, window) form a *group*; every group has storage of its own, sized for its need:

  - "kv" groups hold keys and values in pages of `page_size` positions,
    storage[entry_in_group][page][k|v][kv_head][row][head_dim]; a sequence's pages are listed in the group's page
    table row of its slot. A group with a window only keeps the pages that a query can still see: pages that fall
    wholly behind the window go back to the group's pool while the sequence is still running.
  - "state" groups hold one tensor of fixed shape per entry and slot (float32), zeroed when a slot is taken.

Slots and pages are given back when a sequence ends and are used again; nothing is cleared on reuse except state
(attention never reads beyond a sequence's own length).

Reference: one growing `KVCache` object per sequence with per-layer [positions, kv_heads, head_dim] buffers
(src/etalii_dllm/transformer.py:116-201); its `tokens` list is the per-sequence state.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from .allocators import CacheError, FreeList


@dataclass(frozen=True)
class CacheNeed:
    """What one cache entry needs. kind "kv": keys and values of `kv_heads` x `head_dim` per position, all of them
    (window None) or the last `window`. kind "state": a float32 tensor of `state_shape` per sequence."""

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None
    state_shape: tuple[int, ...] = ()


class KvView:
    """What a kernel needs to address one cache entry."""

    __slots__ = ("base_ptr", "storage", "page_table", "max_pages", "page_size", "kv_heads", "head_dim", "dtype",
                 "window")

    def __init__(self, storage, page_table, page_size, kv_heads, head_dim, window):
        self.storage = storage  # [pages, 2, kv_heads, page_size, head_dim]
        self.base_ptr = storage.data_ptr()
        self.page_table = page_table
        self.max_pages = page_table.shape[1]
        self.page_size = page_size
        self.kv_heads = kv_heads
        self.head_dim = head_dim
        self.dtype = storage.dtype
        self.window = window


class _KvGroup:
    def __init__(self, need: CacheNeed, entries: list[int], n_pages: int, n_slots: int, max_pages: int,
                 page_size: int, dtype, device) -> None:
        self.need, self.entries = need, entries
        self.pool = FreeList(n_pages, "page")
        self.table_host = np.zeros((n_slots, max_pages), dtype=np.int32)
        self.pages_of: list[list[int | None]] = [[] for _ in range(n_slots)]
        self.storage = self.table = None
        if device is not None:
            # zeros, not garbage: a blockwise kernel multiplies masked rows of a page by probability 0
            self.storage = torch.zeros((len(entries), n_pages, 2, need.kv_heads, page_size, need.head_dim),
                                       dtype=dtype, device=device)
            self.table = torch.zeros((n_slots, max_pages), dtype=torch.int32, device=device)
        self.dirty: set[int] = set()


class PagedCache:
    """`needs[i]` is the need of cache entry i (None for an entry without a cache). `max_tokens` is the most tokens
    that live sequences hold together, each sequence rounded up to whole pages; `max_length` bounds one sequence.
    With `device=None` only the host bookkeeping exists (for tests of the accounting)."""

    def __init__(self, needs: Sequence[CacheNeed | None], max_tokens: int, max_length: int, dtype=torch.bfloat16,
                 device=None, page_size: int = 64, max_slots: int | None = None) -> None:
        if max_tokens <= 0 or max_length <= 0:
            raise CacheError("max_tokens and max_length must be positive")
        self.page_size = int(page_size)
        self.max_length = int(max_length)
        self.n_pages = -(-int(max_tokens) // self.page_size)
        self.max_pages = min(self.n_pages, -(-self.max_length // self.page_size))
        self.n_slots = int(max_slots) if max_slots else min(self.n_pages, 1024)
        self.device, self.dtype = device, dtype
        self.slots = FreeList(self.n_slots, "slot")
        self.lengths = [0] * self.n_slots
        self._stage_ring = [[None, None, None] for _ in range(self.STAGING_RING)]  # table rows, indices, event
        self._stage_at = 0
        self.needs = list(needs)
        self._groups: list[_KvGroup] = []
        self._state: dict[int, torch.Tensor | None] = {}
        self._where: dict[int, tuple[_KvGroup, int]] = {}
        by_need: dict[CacheNeed, list[int]] = {}
        for entry, need in enumerate(self.needs):
            if need is None:
                continue
            if need.kind == "kv":
                by_need.setdefault(need, []).append(entry)
            elif need.kind == "state":
                self._state[entry] = None if device is None else torch.zeros(
                    (self.n_slots, *need.state_shape), dtype=torch.float32, device=device)
            else:
                raise CacheError(f"unknown cache kind {need.kind!r}")
        for need, entries in by_need.items():
            pages = self.n_pages
            if need.window:
                # A windowed group holds at most the window (plus the page being filled) per sequence while it
                # decodes; but a whole prompt enters in one step and needs all its positions at once, so there is
                # room for one sequence of the longest length on top of every slot's window.
                per_sequence = -(-need.window // self.page_size) + 1
                pages = min(self.n_pages, per_sequence * self.n_slots + -(-self.max_length // self.page_size))
            group = _KvGroup(need, entries, pages, self.n_slots, self.max_pages, self.page_size, dtype, device)
            self._groups.append(group)
            for index, entry in enumerate(entries):
                self._where[entry] = (group, index)

    # ---- slots ----
    def acquire(self, count: int = 1) -> list[int]:
        """Takes `count` free slots for new sequences (length 0, state zeroed)."""
        slots = self.slots.take(count)
        for slot in slots:
            self.lengths[slot] = 0
            for state in self._state.values():
                if state is not None:
                    state[slot].zero_()
        return slots

    def release(self, slots) -> None:
        """Gives slots and all their pages back."""
        slots = list(slots)
        self.slots.give(slots)
        for slot in slots:
            for group in self._groups:
                group.pool.give(p for p in group.pages_of[slot] if p is not None)
                group.pages_of[slot] = []
            self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    # ---- pages ----
    def reserve(self, slot: int, new_tokens: int) -> None:
        """Makes room for `new_tokens` more positions of the sequence in `slot` (pages are taken as needed)."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not in use")
        end = self.lengths[slot] + new_tokens
        if end > self.max_length:
            raise CacheError(f"sequence of {end} tokens exceeds the cache's longest sequence ({self.max_length})")
        need_pages = -(-end // self.page_size)
        for group in self._groups:
            have = group.pages_of[slot]
            first_needed = 0
            if group.need.window:  # positions below (start + 1 - window) are never read again
                first_needed = max(0, (self.lengths[slot] + 1 - group.need.window)) // self.page_size
                for index in range(min(first_needed, len(have))):
                    if have[index] is not None:
                        group.pool.give([have[index]])
                        have[index] = None
            while len(have) < need_pages:
                index = len(have)
                if index < first_needed:
                    have.append(None)
                    continue
                page = group.pool.take(1)[0]
                have.append(page)
                group.table_host[slot, index] = page
                group.dirty.add(slot)

    def advance(self, slot: int, new_tokens: int) -> None:
        self.lengths[slot] += new_tokens

    def sync_tables(self) -> None:
        """Copies the page-table rows that changed to the device: staged in pinned memory (a small ring, each
        buffer waited for before it is written again), then copied on the current stream without a host wait; a
        few rows go row by row, many through one copy and a scatter."""
        for group in self._groups:
            if group.dirty and group.table is not None:
                rows = sorted(group.dirty)
                width = group.table.shape[1]
                stage, index = self._staging(len(rows), width)
                stage.numpy()[:] = group.table_host[rows]
                if len(rows) <= 4 and group.table.is_cuda:
                    from ..kernels import ops

                    for i, row in enumerate(rows):  # (raw copies: a fraction of the tensor library's dispatch)
                        ops.copy_to_device(group.table.data_ptr() + 4 * row * width, stage.data_ptr() + 4 * i * width,
                                           4 * width)
                elif len(rows) <= 4:
                    for i, row in enumerate(rows):
                        group.table[row].copy_(stage[i], non_blocking=True)
                else:
                    index.numpy()[:] = rows
                    group.table.index_copy_(0, index.to(self.device, non_blocking=True),
                                            stage.to(self.device, non_blocking=True))
                self._staged()
            group.dirty.clear()

    STAGING_RING = 4

    def _staging(self, rows: int, width: int) -> tuple[torch.Tensor, torch.Tensor]:
        entry = self._stage_ring[self._stage_at]
        if entry[2] is not None:
            entry[2].synchronize()
        if entry[0] is None or entry[0].numel() < rows * width:
            entry[0] = torch.empty(max(rows * width, 1024), dtype=torch.int32).pin_memory()
            entry[1] = torch.empty(max(rows, 64), dtype=torch.int64).pin_memory()
        if entry[1].numel() < rows:
            entry[1] = torch.empty(rows, dtype=torch.int64).pin_memory()
        return entry[0][: rows * width].view(rows, width), entry[1][:rows]

    def _staged(self) -> None:
        entry = self._stage_ring[self._stage_at]
        if entry[2] is None:
            entry[2] = torch.cuda.Event()
        entry[2].record()  # (the same event object again and again: recording it anew is all a step needs)
        self._stage_at = (self._stage_at + 1) % self.STAGING_RING

    # ---- views ----
    def kv_view(self, entry: int) -> KvView:
        group, index = self._where[entry]
        return KvView(group.storage[index], group.table, self.page_size, group.need.kv_heads, group.need.head_dim,
                      group.need.window)

    def state(self, entry: int) -> torch.Tensor:
        """The fixed-size state of entry `entry`: [slots, *state_shape] float32."""
        return self._state[entry]

    def groups(self) -> list[tuple[CacheNeed, list[int]]]:
        return [(g.need, list(g.entries)) for g in self._groups]

    def smallest_pool(self) -> int:
        """Pages of the smallest group's pool: what a planner may count on for every group (a windowed group's pool
        is smaller than the cache's page count)."""
        return min((g.pool.count for g in self._groups), default=self.n_pages)

    def pages_held(self) -> int:
        return sum(g.pool.held for g in self._groups)

    def bytes(self) -> int:
        total = sum(g.storage.numel() * g.storage.element_size() for g in self._groups if g.storage is not None)
        return total + sum(s.numel() * 4 for s in self._state.values() if s is not None)

    def check(self) -> None:
        """Accounting invariants: no slot or page lost, held twice, or held by a released slot."""
        self.slots.check()
        for group in self._groups:
            group.pool.check()
            seen: set[int] = set()
            for slot in range(self.n_slots):
                pages = [p for p in group.pages_of[slot] if p is not None]
                assert self.slots.is_held(slot) or not pages, f"released slot {slot} still holds pages"
                for page in pages:
                    assert page not in seen, f"page {page} is held twice"
                    assert group.pool.is_held(page), f"page {page} is in use but marked free"
                    seen.add(page)
            assert len(seen) == group.pool.held, "a page is held by no sequence"

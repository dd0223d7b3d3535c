"""The tokens of one step, as the kernels see them: every sequence's new tokens packed one after another, with each
token's sequence index and absolute position, each sequence's slot and cached length, and the rows whose logits are
wanted. There is no padding: a step runs exactly the tokens it is given."""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch


class StepBatch:
    __slots__ = ("n_seqs", "n_tokens", "n_want", "tokens", "tok_seq", "tok_pos", "cu_seqlens", "slots", "start",
                 "want_rows", "tile_seq", "tile_first", "n_tiles", "h_slots", "h_new", "h_start", "max_new", "max_position", "max_context", "is_decode")


class BatchBuffers:
    """Pinned host staging and device buffers for step metadata: one host-to-device copy per step. A small ring of
    staging buffers lets a step be prepared while the copy of the previous one may still be in flight."""

    RING = 4
    TILE = 64

    def __init__(self, device, capacity: int = 4096) -> None:
        self.device = device
        self.capacity = 0
        self._ring = 0
        self._grow(capacity)

    def _grow(self, capacity: int) -> None:
        self.capacity = capacity
        self.host = [torch.empty(capacity, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.dev = torch.empty(capacity, dtype=torch.int32, device=self.device)
        self.generation = getattr(self, "generation", 0) + 1

    def fill(self, slots: Sequence[int], new_tokens: Sequence[Sequence[int]], starts: Sequence[int],
             want: Sequence[Sequence[int]]) -> StepBatch:
        """`want[b]` lists indices into sequence b's new tokens. Returns the batch with its device views."""
        b = len(slots)
        counts = [len(t) for t in new_tokens]
        n = sum(counts)
        r = sum(len(w) for w in want)
        # tiles of up to TILE new tokens of one sequence for the prefill attention, the longest contexts first
        tiles = [(i, first) for i, c in enumerate(counts) for first in range(0, c, self.TILE)]
        tiles.sort(key=lambda t: -(starts[t[0]] + t[1]))
        nt = len(tiles)
        total = 3 * n + (b + 1) + 2 * b + r + 2 * nt
        if total > self.capacity:
            self._grow(max(total, 2 * self.capacity))
        ring = self._ring
        self._ring = (ring + 1) % self.RING
        if self.events[ring] is not None:
            self.events[ring].synchronize()
        host = self.host[ring].numpy()
        cu = np.zeros(b + 1, dtype=np.int32)
        np.cumsum(counts, out=cu[1:])
        o = 0
        host[o:o + n] = np.concatenate([np.asarray(seq) for seq in new_tokens]) if n else np.zeros(0, np.int32); o += n
        host[o:o + n] = np.repeat(np.arange(b, dtype=np.int32), counts); o += n
        pos = np.concatenate([np.arange(s, s + c, dtype=np.int32) for s, c in zip(starts, counts)]) if n else \
            np.zeros(0, np.int32)
        host[o:o + n] = pos; o += n
        host[o:o + b + 1] = cu; o += b + 1
        host[o:o + b] = np.asarray(slots, dtype=np.int32); o += b
        host[o:o + b] = np.asarray(starts, dtype=np.int32); o += b
        rows = [cu[i] + w for i, ws in enumerate(want) for w in ws]
        host[o:o + r] = np.asarray(rows, dtype=np.int32) if r else np.zeros(0, np.int32); o += r
        host[o:o + nt] = [t[0] for t in tiles]; o += nt
        host[o:o + nt] = [t[1] for t in tiles]; o += nt
        self.dev[:total].copy_(self.host[ring][:total], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[ring] = event

        batch = StepBatch()
        batch.n_seqs, batch.n_tokens, batch.n_want = b, n, r
        o = 0
        batch.tokens = self.dev[o:o + n]; o += n
        batch.tok_seq = self.dev[o:o + n]; o += n
        batch.tok_pos = self.dev[o:o + n]; o += n
        batch.cu_seqlens = self.dev[o:o + b + 1]; o += b + 1
        batch.slots = self.dev[o:o + b]; o += b
        batch.start = self.dev[o:o + b]; o += b
        batch.want_rows = self.dev[o:o + r]; o += r
        batch.tile_seq = self.dev[o:o + nt]; o += nt
        batch.tile_first = self.dev[o:o + nt]; o += nt
        batch.n_tiles = nt
        batch.h_slots, batch.h_new, batch.h_start = list(slots), counts, list(starts)
        batch.max_new = max(counts) if counts else 0
        batch.max_context = max((s + c for s, c in zip(starts, counts)), default=0)
        batch.max_position = batch.max_context - 1
        batch.is_decode = all(c == 1 for c in counts)
        return batch

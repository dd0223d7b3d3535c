"""The tokens of one step, as the kernels see them: every sequence's new tokens packed one after another, with each
token's sequence index and absolute position, each sequence's slot and cached length, and the rows whose logits are
wanted. There is no padding: a step runs exactly the tokens it is given.

`StepLayout` is the one place that says which fields a step's metadata has and where each lies in the step's int32
buffer; `step_values` computes them on the host. The step function (`BatchBuffers.fill`) and the captured decode
step (`DecodeGraph`) both lay their buffers out with it, so a part that needs one more field per token or per
sequence registers it once (`register_step_field`) and finds it as `batch.<name>` on both paths."""
from __future__ import annotations

from typing import Callable, Sequence

import numpy as np
import torch

TILE = 64
"""New tokens of one sequence per tile of the prefill attention."""

_PER = ("token", "sequence", "sequence+1", "want", "tile", "one")
FIELDS: list[tuple[str, str]] = [
    ("tokens", "token"), ("tok_seq", "token"), ("tok_pos", "token"), ("cu_seqlens", "sequence+1"),
    ("slots", "sequence"), ("start", "sequence"), ("want_rows", "want"), ("tile_seq", "tile"), ("tile_first", "tile"),
]
"""(name, one value per ...) of the fields every step has, in buffer order."""
_EXTRA: dict[str, tuple[str, Callable]] = {}


def register_step_field(name: str, per: str, values: Callable[["StepInfo"], np.ndarray]) -> None:
    """Adds an int32 field to every step's metadata: `per` is "token" or "sequence", `values(info)` returns the
    field's values from the host-side description of the step (`info.slots`, `info.counts`, `info.starts`). The
    field arrives on the device with the step's one copy and is found as `batch.<name>`. In a captured decode run
    the field keeps the values it had when the run was loaded unless the part's own kernel advances it."""
    if per not in ("token", "sequence"):
        raise ValueError("a step field has one value per token or per sequence")
    if name in _EXTRA or any(name == known for known, _ in FIELDS) or name in StepBatch.HOST_FIELDS:
        raise ValueError(f"step field {name!r} exists already")
    _EXTRA[name] = (per, values)


def unregister_step_field(name: str) -> None:
    _EXTRA.pop(name, None)


class StepInfo:
    """The host-side description of a step that field functions see."""

    def __init__(self, slots, counts, starts) -> None:
        self.slots, self.counts, self.starts = list(slots), list(counts), list(starts)


class StepBatch:
    """A step as the parts see it: the device views of the layout's fields as attributes, and the host-side counts."""

    HOST_FIELDS = ("n_seqs", "n_tokens", "n_want", "n_tiles", "h_slots", "h_new", "h_start", "max_new",
                   "max_position", "max_context", "is_decode")


class StepLayout:
    """Where each field of a step with these counts lies in the step's int32 buffer. `extra` appends fields that
    only one user of the layout has (the decode run's step counter)."""

    def __init__(self, n_tokens: int, n_seqs: int, n_want: int, n_tiles: int, extra: Sequence[tuple[str, str]] = ()):
        sizes = {"token": n_tokens, "sequence": n_seqs, "sequence+1": n_seqs + 1, "want": n_want, "tile": n_tiles,
                 "one": 1}
        self.counts = (n_tokens, n_seqs, n_want, n_tiles)
        self.offsets: dict[str, tuple[int, int]] = {}
        at = 0
        for name, per in (*FIELDS, *((name, per) for name, (per, _) in _EXTRA.items()), *extra):
            self.offsets[name] = (at, sizes[per])
            at += sizes[per]
        self.total = at

    def view(self, buffer, name: str):
        begin, count = self.offsets[name]
        return buffer[begin:begin + count]

    def write(self, host: np.ndarray, values: dict[str, np.ndarray]) -> None:
        for name, value in values.items():
            begin, count = self.offsets[name]
            host[begin:begin + count] = value

    def attach(self, batch: StepBatch, device_buffer: torch.Tensor) -> None:
        """Sets every field's device view on `batch`."""
        for name in self.offsets:
            setattr(batch, name, self.view(device_buffer, name))


def prefill_tiles(counts: Sequence[int], starts: Sequence[int]) -> list[tuple[int, int]]:
    """Tiles of up to TILE new tokens of one sequence for the prefill attention, the longest contexts first."""
    tiles = [(i, first) for i, c in enumerate(counts) for first in range(0, c, TILE)]
    tiles.sort(key=lambda t: -(starts[t[0]] + t[1]))
    return tiles


def step_values(slots: Sequence[int], new_tokens: Sequence[Sequence[int]], starts: Sequence[int],
                want: Sequence[Sequence[int]], tiles: Sequence[tuple[int, int]] = ()) -> dict[str, np.ndarray]:
    """The values of every field of a step, by name."""
    b = len(slots)
    counts = [len(t) for t in new_tokens]
    n = sum(counts)
    cu = np.zeros(b + 1, dtype=np.int32)
    np.cumsum(counts, out=cu[1:])
    empty = np.zeros(0, np.int32)
    values = {
        "tokens": np.concatenate([np.asarray(seq, dtype=np.int32) for seq in new_tokens]) if n else empty,
        "tok_seq": np.repeat(np.arange(b, dtype=np.int32), counts),
        "tok_pos": np.concatenate([np.arange(s, s + c, dtype=np.int32) for s, c in zip(starts, counts)]) if n
        else empty,
        "cu_seqlens": cu,
        "slots": np.asarray(slots, dtype=np.int32),
        "start": np.asarray(starts, dtype=np.int32),
        "want_rows": np.asarray([cu[i] + w for i, ws in enumerate(want) for w in ws], dtype=np.int32),
        "tile_seq": np.asarray([t[0] for t in tiles], dtype=np.int32),
        "tile_first": np.asarray([t[1] for t in tiles], dtype=np.int32),
    }
    if _EXTRA:
        info = StepInfo(slots, counts, starts)
        for name, (_, function) in _EXTRA.items():
            values[name] = np.asarray(function(info), dtype=np.int32)
    return values


class BatchBuffers:
    """Pinned host staging and device buffers for step metadata: one host-to-device copy per step. A small ring of
    staging buffers lets a step be prepared while the copy of the previous one may still be in flight."""

    RING = 4
    TILE = TILE

    def __init__(self, device, capacity: int = 4096) -> None:
        self.device = device
        self.capacity = 0
        self._ring = 0
        self._grow(capacity)

    def _grow(self, capacity: int) -> None:
        self.capacity = capacity
        self.host = [torch.empty(capacity, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.host_arrays = [h.numpy() for h in self.host]  # (views, made once: a step costs no object for them)
        self.events = [None] * self.RING
        self.dev = torch.empty(capacity, dtype=torch.int32, device=self.device)
        self.generation = getattr(self, "generation", 0) + 1

    def fill(self, slots: Sequence[int], new_tokens: Sequence[Sequence[int]], starts: Sequence[int],
             want: Sequence[Sequence[int]]) -> StepBatch:
        """`want[b]` lists indices into sequence b's new tokens. Returns the batch with its device views."""
        counts = [len(t) for t in new_tokens]
        tiles = prefill_tiles(counts, starts)
        layout = StepLayout(sum(counts), len(slots), sum(len(w) for w in want), len(tiles))
        if layout.total > self.capacity:
            self._grow(max(layout.total, 2 * self.capacity))
        ring = self._ring
        self._ring = (ring + 1) % self.RING
        if self.events[ring] is not None:
            self.events[ring].synchronize()
        layout.write(self.host_arrays[ring], step_values(slots, new_tokens, starts, want, tiles))
        if self.dev.is_cuda:
            from ..kernels import ops

            ops.copy_to_device(self.dev.data_ptr(), self.host[ring].data_ptr(), 4 * layout.total)
            if self.events[ring] is None:
                self.events[ring] = torch.cuda.Event()
            self.events[ring].record()  # (the staging buffer is free again when this has passed)
        else:
            self.dev[:layout.total].copy_(self.host[ring][:layout.total])

        batch = StepBatch()
        layout.attach(batch, self.dev)
        batch.n_tokens, batch.n_seqs, batch.n_want, batch.n_tiles = layout.counts
        batch.h_slots, batch.h_new, batch.h_start = list(slots), counts, list(starts)
        batch.max_new = max(counts) if counts else 0
        batch.max_context = max((s + c for s, c in zip(starts, counts)), default=0)
        batch.max_position = batch.max_context - 1
        batch.is_decode = all(c == 1 for c in counts)
        return batch

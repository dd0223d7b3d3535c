"""What the parts share at run time: the device, the activation dtype, reusable work buffers and device copies of
weights and tables."""
from __future__ import annotations

from typing import Callable

import torch


class Workspace:
    """Named work buffers that are allocated once and reused by every step. A buffer grows when a larger one is
    asked for; `generation` counts such reallocations (captured CUDA graphs hold the old addresses and are dropped
    when it changes)."""

    def __init__(self, device) -> None:
        self.device = device
        self.generation = 0
        self._buffers: dict[str, torch.Tensor] = {}
        self._views: dict[tuple, torch.Tensor] = {}

    def buffer(self, name: str, shape, dtype) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        view = self._views.get(key)  # the same step shapes come again and again: the view object is kept
        if view is not None:
            return view
        count = 1
        for d in shape:
            count *= int(d)
        have = self._buffers.get(name)
        if have is None or have.dtype != dtype or have.numel() < count:
            capacity = max(count, 1) if have is None or have.dtype != dtype else max(count, 2 * have.numel())
            have = torch.empty(capacity, dtype=dtype, device=self.device)
            self._buffers[name] = have
            self.generation += 1
            self._views = {k: v for k, v in self._views.items() if k[0] != name}
        if len(self._views) > 4096:
            self._views.clear()
        view = have[:count].view(*shape)
        self._views[key] = view
        return view

    def zeros(self, name: str, count: int, dtype) -> torch.Tensor:
        """A buffer that starts as zeros and is kept between steps (kernels that use it leave it zero)."""
        have = self._buffers.get(name)
        if have is None or have.dtype != dtype or have.numel() < count:
            have = torch.zeros(max(count, 256), dtype=dtype, device=self.device)
            self._buffers[name] = have
            self.generation += 1
        return have[:count]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._buffers.values())


class Runtime:
    def __init__(self, device, dtype: torch.dtype, max_length: int) -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError(f"device {device!r}: this library runs on CUDA devices only (there is no CPU path)")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported (bfloat16 and float32 are)")
        self.dtype = dtype
        self.max_length = int(max_length)
        self.ws = Workspace(self.device)
        self._device_copies: dict[tuple[int, torch.dtype], torch.Tensor] = {}
        self._shared: dict = {}
        self._keep: list = []

    def to_device(self, tensor: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
        """A device copy of a loaded tensor in `dtype`; the same source tensor is uploaded once (a tied head and
        the embedding share their copy)."""
        dtype = dtype or tensor.dtype
        key = (id(tensor), dtype)
        found = self._device_copies.get(key)
        if found is None:
            found = tensor.to(device=self.device, dtype=dtype).contiguous()
            self._device_copies[key] = found
            self._keep.append(tensor)  # keeps id() unique while the copy is cached
        return found

    def shared(self, key, make: Callable[[], torch.Tensor]) -> torch.Tensor:
        """One device object per key (rotary tables shared by all layers with the same parameters)."""
        if key not in self._shared:
            self._shared[key] = make()
        return self._shared[key]

    def done_loading(self) -> None:
        self._device_copies.clear()
        self._keep.clear()

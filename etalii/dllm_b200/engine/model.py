"""A model put together from a `ModelSpec`: parts built from the registries, weights bound by name, a cache sized for
what the mixers ask for, and the forward pass of one step over a packed batch."""
from __future__ import annotations

from typing import Mapping

import torch

from ..cache.paged import PagedCache
from ..parts.registry import build_part, part_factory
from ..parts.spec import ModelSpec
from .runtime import Runtime


class UnsupportedConfiguration(ValueError):
    """A configuration that loads but that the kernels of one of its parts cannot run; the message names the rule."""


class Model:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], rt: Runtime, max_tokens: int,
                 max_slots: int | None = None, page_size: int = 64) -> None:
        self.spec, self.rt = spec, rt
        self.vocab_size, self.hidden_size = spec.vocab_size, spec.hidden_size

        # every part is built first and asked whether it can run here (`supports(rt)`: None, or the reason why
        # not); only then do weights go to the device
        built: list[tuple[str, object, object]] = []

        def build(path, role, part_spec):
            part = build_part(role, part_spec)
            built.append((path, part, part_spec))
            return part

        self.embedding = build("embedding", "embedding", spec.embedding)
        layer_parts = []
        for index, layer in enumerate(spec.layers):
            roles = layer.roles()
            layer_parts.append({name: build(f"layers.{index}.{name}", roles[name], part_spec)
                                for name, part_spec in layer.parts.items()})
        self.final_norm = build("final_norm", "norm", spec.final_norm)
        self.head = build("head", "head", spec.head)
        refused = []
        for path, part, _ in built:
            reason = part.supports(rt) if hasattr(part, "supports") else None
            if reason:
                refused.append(f"{path}: {reason}")
        if refused:
            raise UnsupportedConfiguration("this configuration cannot run on the kernels:\n  " + "\n  ".join(refused))
        for _, part, part_spec in built:
            part.bind({local: tensors[name] for local, name in part_spec.names.items()}, rt)
        self.blocks = [part_factory("block", layer.block)(**parts) for layer, parts in zip(spec.layers, layer_parts)]
        rt.done_loading()
        if torch.device(rt.device).type == "cuda":  # what the parts say they call, compiled side by side
            from ..kernels.build import prebuild

            names = {"elementwise", "gemm_simt" if rt.dtype == torch.float32 else "gemv"}
            for part in self._layer_parts():
                if hasattr(part, "kernel_libraries"):
                    names |= set(part.kernel_libraries(rt))
            prebuild(sorted(names))

        self.order = spec.run_order()
        n_entries = max((e.cache for e in self.order), default=-1) + 1
        needs = [None] * n_entries
        for entry in self.order:
            if entry.writes_cache:
                mixer = self.blocks[entry.layer].mixer
                needs[entry.cache] = mixer.cache_need() if hasattr(mixer, "cache_need") else None
        self.cache = PagedCache(needs, max_tokens=max_tokens, max_length=rt.max_length, dtype=rt.dtype,
                                device=rt.device, page_size=page_size, max_slots=max_slots)
        self._views = []
        for entry in self.order:
            need = needs[entry.cache]
            if need is None:
                self._views.append(None)
            elif need.kind == "kv":
                self._views.append(self.cache.kv_view(entry.cache))
            else:
                self._views.append(self.cache.state(entry.cache))

        self._plan_prefetch()
        # the C++ host side of prefill-sized steps, for models made of the parts it restates (else None)
        from ..kernels.launcher import PreNormLayers

        self.native_layers = PreNormLayers.build(self) if torch.device(rt.device).type == "cuda" else None
        if self.native_layers is not None:
            from ..kernels.build import prebuild

            prebuild(sorted(self.native_layers.libraries()))

    def _layer_parts(self, block=None):
        """The parts of one block, or of all blocks: a block's `parts` mapping where it has one, else what it holds
        under the names its class declares."""
        for b in (self.blocks if block is None else [block]):
            parts = getattr(b, "parts", None)
            if parts is None:
                parts = {name: getattr(b, name) for name in getattr(type(b), "PARTS", {}) if hasattr(b, name)}
            yield from parts.values()

    def capturable(self) -> bool:
        """Whether a decode step of this model can be captured in a CUDA graph: every block and part may say no
        (`CAPTURABLE = False`, e.g. a part written with allocating torch ops); the library's own all can."""
        things = [*self.blocks, *self._layer_parts(), self.embedding, self.final_norm, self.head]
        return all(getattr(thing, "CAPTURABLE", True) for thing in things)

    def _plan_prefetch(self, ahead: int = 4) -> None:
        """Tells the decode-sized products which weights come `ahead` products later in the run order, so that they
        can be brought into L2 before they are needed (kernels/ops.py::prefetch_hints)."""
        from ..kernels import ops

        order = []
        for entry in self.order:
            for part in self._layer_parts(self.blocks[entry.layer]):
                order += [v for v in vars(part).values()
                          if isinstance(v, torch.Tensor) and v.dim() == 2 and v.dtype == torch.bfloat16]
        order += [v for v in vars(self.head).values() if isinstance(v, torch.Tensor) and v.dim() == 2
                  and v.dtype == torch.bfloat16]
        self._prefetch = {}
        for index, tensor in enumerate(order[:-ahead] if len(order) > ahead else []):
            self._prefetch[tensor.data_ptr()] = order[index + ahead]
        # A last matrix too large for one request (the head's) but well inside L2 is asked for in slices of its rows
        # by the products before it, one slice each.
        last = order[-1] if len(order) > ahead else None
        if last is not None and ops.PREFETCH_LIMIT < last.numel() * last.element_size() <= ops.PREFETCH_SLICED_LIMIT:
            pieces = min(2 * ahead, len(order) - 1)
            rows = -(-last.shape[0] // pieces)
            for index, tensor in enumerate(order[-1 - pieces:-1]):
                self._prefetch[tensor.data_ptr()] = last[index * rows:(index + 1) * rows]

    def forward(self, batch, greedy_out: torch.Tensor | None = None) -> torch.Tensor:
        """Runs the batch's tokens through every scheduled layer; returns float32 logits [wanted rows, vocab]
        (None when no row is wanted: the cache is still filled). With `greedy_out` (int32 [wanted rows]) a head
        that can make the greedy choice inside its product writes the chosen tokens there and no logits are
        computed: the return value is then None."""
        from ..kernels import ops

        rt = self.rt
        ops.prefetch_hints = self._prefetch  # this model's hints (they live and die with the model)
        x = self.embedding.forward(batch.tokens, batch.n_tokens, rt)
        if self.native_layers is not None and self.native_layers.takes(batch):
            self.native_layers.run(x, batch, rt)  # every layer's launches from one C++ call
        else:
            for entry, view in zip(self.order, self._views):
                self.blocks[entry.layer].forward(x, batch, view, rt, entry.writes_cache)
        if batch.n_want == 0:
            return None
        if batch.is_decode and batch.n_want == batch.n_tokens and hasattr(self.final_norm, "lazy") \
                and getattr(self.head, "accepts_pending_norm", False):
            pending = self.final_norm.lazy(x, rt)  # every row is wanted, in order: no gather
            if greedy_out is not None and hasattr(self.head, "choose_greedy") and \
                    self.head.choose_greedy(pending, rt, greedy_out):
                return None
            return self.head.forward(pending, rt)
        hidden = self.final_norm.forward(x, rt, rows=batch.want_rows, n_rows=batch.n_want, name="final_hidden")
        return self.head.forward(hidden, rt)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for part in self._layer_parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                    seen.add(value.data_ptr())
                    total += value.numel() * value.element_size()
        for part in (self.embedding, self.final_norm, self.head):
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                    seen.add(value.data_ptr())
                    total += value.numel() * value.element_size()
        return total

"""What a model is made of, as data: parts with their sizes and constants, layer by layer, and the order they run in.

An architecture's `build_spec(config)` returns a `ModelSpec`. Nothing below knows which model it describes: a
`PartSpec` names a registered kind ("rmsnorm", "attention", "swiglu", ...) and carries that part's parameters; a
`LayerSpec` puts a mixer, a feed-forward and their norms into a block arrangement; `schedule` lists which layer runs
when and with which cache, so a layer may run twice or read the cache another layer wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part owns. `init` tells the random-weights mode how to fill it: "normal" ~ N(0, std),
    "ones" ~ 1 + N(0, std / 2) (norm weights), "int" for integer tables (kept as int32)."""

    shape: tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    names: Mapping[str, str] = field(default_factory=dict)
    """The part's own parameter name -> the tensor's name in the checkpoint."""


@dataclass(frozen=True)
class LayerSpec:
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: str = "pre_norm"
    """The arrangement: "pre_norm" is x += mixer(norm(x)); x += feed_forward(norm(x))."""


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. `cache` is the index of the cache entry the mixer uses; with `writes_cache` False the
    mixer only reads it (it was written earlier in the same step by the entry that owns it)."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    max_position: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    final_norm: PartSpec
    head: PartSpec
    schedule: tuple[ScheduleEntry, ...] = ()
    """Empty means every layer once, in order, each with a cache of its own."""
    stop_token_ids: tuple[int, ...] = ()
    equal_if_present: Mapping[str, str] = field(default_factory=dict)
    """Checkpoint tensors that may be present although the model does not use them, and must then equal another
    tensor (a tied model that also stores its head)."""
    ignored_suffixes: tuple[str, ...] = ()
    """Checkpoint tensors with these endings are skipped (stored rotary tables)."""

    def run_order(self) -> tuple[ScheduleEntry, ...]:
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i, i) for i in range(len(self.layers)))

    def part_specs(self) -> list[tuple[str, str, PartSpec]]:
        """Every part as (path in the model, role, spec), e.g. ("layers.2.mixer", "mixer", ...)."""
        out = [("embedding", "embedding", self.embedding)]
        for index, layer in enumerate(self.layers):
            out += [
                (f"layers.{index}.mixer_norm", "norm", layer.mixer_norm),
                (f"layers.{index}.mixer", "mixer", layer.mixer),
                (f"layers.{index}.feed_forward_norm", "norm", layer.feed_forward_norm),
                (f"layers.{index}.feed_forward", "feed_forward", layer.feed_forward),
            ]
        out += [("final_norm", "norm", self.final_norm), ("head", "head", self.head)]
        return out

"""What a model is made of, as data: parts with their sizes and constants, layer by layer, and the order they run in.

An architecture's `build_spec(config)` returns a `ModelSpec`. Nothing below knows which model it describes: a
`PartSpec` names a registered kind ("rmsnorm", "attention", "swiglu", ...) and carries that part's parameters; a
`LayerSpec` names a block arrangement and gives it its parts by name (the arrangement says which names it wants and
which role each plays); `schedule` lists which layer runs when and with which cache, so a layer may run twice or
read the cache another layer wrote.
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


@dataclass(frozen=True, init=False)
class LayerSpec:
    """One layer: `block` names a registered arrangement, `parts` maps the names that arrangement asks for (its
    class attribute `PARTS`: name -> role) to the specs of the parts. The pre-norm arrangement asks for `mixer`,
    `feed_forward`, `mixer_norm` and `feed_forward_norm`, which may also be given as the first four arguments;
    another arrangement (norms behind the parts as well, one norm for both parts) names its own."""

    block: str
    parts: Mapping[str, PartSpec]

    def __init__(self, mixer: PartSpec | None = None, feed_forward: PartSpec | None = None,
                 mixer_norm: PartSpec | None = None, feed_forward_norm: PartSpec | None = None,
                 block: str = "pre_norm", parts: Mapping[str, PartSpec] | None = None) -> None:
        named = dict(parts or {})
        for name, spec in (("mixer", mixer), ("feed_forward", feed_forward), ("mixer_norm", mixer_norm),
                           ("feed_forward_norm", feed_forward_norm)):
            if spec is not None:
                if name in named:
                    raise ValueError(f"the layer's part {name!r} is given twice")
                named[name] = spec
        object.__setattr__(self, "block", block)
        object.__setattr__(self, "parts", named)

    def roles(self) -> dict[str, str]:
        """name -> role of this layer's parts, as its arrangement declares them; the names must match exactly."""
        from .registry import part_factory

        wanted = dict(getattr(part_factory("block", self.block), "PARTS"))
        if set(wanted) != set(self.parts):
            raise ValueError(f"block {self.block!r} takes the parts {sorted(wanted)}; the layer gives "
                             f"{sorted(self.parts)}")
        return wanted


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
            roles = layer.roles()
            out += [(f"layers.{index}.{name}", roles[name], spec) for name, spec in layer.parts.items()]
        out += [("final_norm", "norm", self.final_norm), ("head", "head", self.head)]
        return out

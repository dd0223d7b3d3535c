"""Registries of part kinds. A part class is registered under a role ("norm", "position", "mixer", "feed_forward",
"block", "embedding", "head") and a kind name; `build_part` makes an instance from a `PartSpec`."""
from __future__ import annotations

from typing import Any, Callable

ROLES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_PARTS: dict[str, dict[str, Callable[..., Any]]] = {role: {} for role in ROLES}


def register_part(role: str, kind: str, factory: Callable[..., Any], replace: bool = False) -> None:
    if role not in _PARTS:
        raise ValueError(f"unknown role {role!r} (roles: {', '.join(ROLES)})")
    if kind in _PARTS[role] and not replace:
        raise ValueError(f"{role} {kind!r} is already registered")
    _PARTS[role][kind] = factory


def unregister_part(role: str, kind: str) -> None:
    _PARTS[role].pop(kind, None)


def part_factory(role: str, kind: str) -> Callable[..., Any]:
    found = _PARTS[role].get(kind)
    if found is None:
        raise ValueError(f"no {role} of kind {kind!r} (registered: {', '.join(sorted(_PARTS[role])) or 'none'})")
    return found


def build_part(role: str, spec: Any) -> Any:
    """An instance of the registered class for `spec.kind`, built from `spec.params`."""
    return part_factory(role, spec.kind)(**dict(spec.params))

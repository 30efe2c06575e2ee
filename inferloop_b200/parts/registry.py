"""Registries from a spec's `kind` to the class that implements it, one per role."""
from __future__ import annotations

from typing import Callable, Dict, Type

from ..config.spec import PartSpec
from .base import BuildContext, Part

ROLES = ("norm", "position", "mixer", "feed_forward", "block", "logits")
_REGISTRY: Dict[str, Dict[str, Type[Part]]] = {r: {} for r in ROLES}


def register(role: str, kind: str, cls: Type[Part], replace: bool = False) -> None:
    if role not in _REGISTRY:
        raise KeyError(f"unknown part role {role!r}; roles are {ROLES}")
    if kind in _REGISTRY[role] and not replace:
        raise KeyError(f"{role} kind {kind!r} is already registered")
    _REGISTRY[role][kind] = cls


def unregister(role: str, kind: str) -> None:
    _REGISTRY[role].pop(kind, None)


def kinds(role: str):
    _ensure_builtin()
    return sorted(_REGISTRY[role])


def build(role: str, spec: PartSpec, ctx: BuildContext, prefix: str = "") -> Part:
    _ensure_builtin()
    try:
        cls = _REGISTRY[role][spec.kind]
    except KeyError:
        raise KeyError(
            f"no {role} of kind {spec.kind!r} is registered (known: {sorted(_REGISTRY[role])})") from None
    return cls(spec, ctx, prefix)


def build_norm(spec: PartSpec, ctx: BuildContext, prefix: str, width: int) -> Part:
    """A norm needs the width of what it normalises, which its owner knows."""
    _ensure_builtin()
    try:
        cls = _REGISTRY["norm"][spec.kind]
    except KeyError:
        raise KeyError(f"no norm of kind {spec.kind!r} is registered") from None
    return cls(spec, ctx, prefix, width=width)


def build_block(layer, ctx: BuildContext, prefix: str) -> Part:
    """A block is built from the whole layer spec: it builds its own parts."""
    _ensure_builtin()
    try:
        cls = _REGISTRY["block"][layer.block.kind]
    except KeyError:
        raise KeyError(f"no block of kind {layer.block.kind!r} is registered") from None
    return cls(layer.block, ctx, prefix, layer=layer)


_BUILTIN_DONE = False


def _ensure_builtin() -> None:
    global _BUILTIN_DONE
    if _BUILTIN_DONE:
        return
    _BUILTIN_DONE = True
    from . import attention, block, logits, mlp, norm, rope  # noqa: F401  (they register themselves)

"""Registries of part kinds.  A recipe names parts by (slot, kind); anything registered
here - by the framework or by a user's own module - can be built without touching the
framework's files."""

from __future__ import annotations

from typing import Callable

import torch

from ..config.recipe import PartSpec

SLOTS = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, Callable]] = {s: {} for s in SLOTS}


def register_part(slot: str, kind: str, factory: Callable | None = None):
    """`register_part("mixer", "my_mixer", MyMixer)` or as a class decorator."""
    if slot not in _REGISTRY:
        raise ValueError(f"unknown part slot {slot!r}; slots: {', '.join(SLOTS)}")

    def _do(f: Callable) -> Callable:
        _REGISTRY[slot][kind] = f
        return f

    return _do(factory) if factory is not None else _do


def registered_parts(slot: str) -> list[str]:
    return sorted(_REGISTRY[slot])


def build_part(slot: str, spec: PartSpec, dtype: torch.dtype, device: torch.device, **extra):
    try:
        factory = _REGISTRY[slot][spec.kind]
    except KeyError:
        raise ValueError(
            f"no {slot} part of kind {spec.kind!r}; registered: {', '.join(registered_parts(slot)) or '(none)'}") from None
    return factory(spec, dtype, device, **extra)


def build_block(layer, dtype: torch.dtype, device: torch.device):
    """Blocks are built from the whole `LayerSpec` (they build their own mixer, feed-forward and norms)."""
    try:
        factory = _REGISTRY["block"][layer.block]
    except KeyError:
        raise ValueError(
            f"no block arrangement {layer.block!r}; registered: {', '.join(registered_parts('block')) or '(none)'}") from None
    return factory(layer, dtype, device)

"""One registry from an architecture's name to its configuration class and recipe.

The reference has no registry (its loader accepts `model_type == "llama"` only,
model/llama.py:41-42); here a model folder's config.json picks the entry by
`architectures[0]`, falling back to `model_type`, and an unknown name is an error that
lists what is registered.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .files import ConfigError
from .recipe import ModelRecipe


@dataclass(frozen=True)
class Architecture:
    name: str                      # config.json "architectures"[0]
    model_type: str                # config.json "model_type"
    config_from_hf: Callable[[dict[str, Any], dict[str, Any] | None], Any]
    recipe: Callable[[Any], ModelRecipe]


_BY_NAME: dict[str, Architecture] = {}
_BY_MODEL_TYPE: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    if arch.name in _BY_NAME and _BY_NAME[arch.name] is not arch:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _BY_NAME[arch.name] = arch
    _BY_MODEL_TYPE.setdefault(arch.model_type, arch)
    return arch


def registered_architectures() -> list[str]:
    return sorted(_BY_NAME)


def resolve_architecture(cfg: dict[str, Any]) -> Architecture:
    """The entry that a config.json asks for."""
    names = cfg.get("architectures") or []
    for n in names:
        if n in _BY_NAME:
            return _BY_NAME[n]
    mt = cfg.get("model_type")
    if not names and mt in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[mt]
    asked = names[0] if names else f"model_type={mt!r}"
    raise ConfigError(
        f"unknown architecture {asked!r}; registered: {', '.join(registered_architectures()) or '(none)'}")

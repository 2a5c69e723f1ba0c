"""The data that describes a model to the rest of the framework.

An architecture turns its typed configuration into a `ModelRecipe`: one `LayerSpec` per
layer, each naming its mixer, feed-forward, norms and arrangement by registry key with
every size and constant as a parameter, and an `order` list that says which layer runs
when and on which cache lane. Nothing below the recipe knows what model it belongs to.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by registry key, with its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "params", MappingProxyType(dict(self.params)))

    def __getitem__(self, key: str) -> Any:
        return self.params[key]


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (`block`) of a mixer, a feed-forward and their norms.

    `prefix` is the layer's part of every tensor name ("model.layers.3."); `names` maps
    the arrangement's slots ("mixer", "feed_forward", "norm_mixer", "norm_feed_forward")
    to the sub-prefix used in the checkpoint ("self_attn.", "input_layernorm.", ...).
    """

    block: str
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec
    names: Mapping[str, str]

    def __post_init__(self) -> None:
        object.__setattr__(self, "names", MappingProxyType(dict(self.names)))


@dataclass(frozen=True)
class Run:
    """One entry of the execution order.

    `layer` indexes `ModelRecipe.layers` (a layer may be named more than once).
    `lane` is the cache lane the mixer works on; lanes are numbered by the recipe and a
    lane's geometry comes from the first run that writes it.  A run with `writes=False`
    reads a lane that an earlier run of the same step has written (cache sharing).
    """

    layer: int
    lane: int
    writes: bool = True


@dataclass(frozen=True)
class ModelRecipe:
    architecture: str
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[Run, ...]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    vocab_size: int
    hidden_size: int
    max_positions: int
    eos_token_ids: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        written: set[int] = set()
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {run.layer}, but there are {len(self.layers)}")
            if run.writes:
                if run.lane in written:
                    raise ValueError(f"order[{i}] writes cache lane {run.lane}, which an earlier run already writes")
                written.add(run.lane)
            elif run.lane not in written:
                raise ValueError(f"order[{i}] reads cache lane {run.lane} before any run has written it")
        lanes = sorted(written)
        if lanes != list(range(len(lanes))):
            raise ValueError(f"cache lanes must be numbered 0..n-1, got {lanes}")

    @property
    def num_lanes(self) -> int:
        return len({r.lane for r in self.order})

"""What every part is: a thing built from a `PartSpec`, that names the weights it needs and
receives them by those names.  A part never learns which model it sits in."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.recipe import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part wants from the checkpoint.

    rule: "compute" - floating matrix used in matrix products, cast to the run's dtype;
          "float32" - small floating tensor (a norm gain) that is held in float32 in every mode;
          "int32"   - an integer table.
    init: how the random-weights mode fills it: "normal" N(0, std), "gain" 1 + N(0, 0.1).
    alias: a full tensor name to use instead when this one is absent from the checkpoint
           (a head tied to the embedding).
    """

    shape: tuple[int, ...]
    rule: str = "compute"
    init: str = "normal"
    std: float = 0.02
    alias: str | None = None


class Part:
    """Base of mixers, feed-forwards, norms, position encodings, embeddings and heads."""

    def __init__(self, spec: PartSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.spec = spec
        self.dtype = dtype
        self.device = device

    def weight_specs(self) -> dict[str, WeightSpec]:
        """Names (relative to the part's prefix) and shapes of the tensors this part needs."""
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receives the tensors named by `weight_specs`, already on the device and cast."""

    # ---- optional: folding the norms into products (a decode step's mixers and feed-forwards) ----
    def takes_row_scaled(self, n_tokens: int) -> bool:
        """True when `forward` may be given its input as an `ops.RowScaled` (normed activations whose
        per-row scale the part's first product applies) in a step of `n_tokens` tokens."""
        return False

    def feeds_norm_sink(self, n_tokens: int) -> bool:
        """True when `forward` takes `sink=ops.NormSink(...)` in such a step: its last product then adds
        its output to the residual stream itself and returns an `ops.RowScaled` for the norm that follows."""
        return False


@dataclass(frozen=True)
class CacheNeed:
    """Paged key/value storage a mixer wants: per token `kv_heads * head_dim` keys and as many
    values; `window` > 0 means only the last `window` positions are ever read."""

    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state a mixer wants (one slot per live request)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32

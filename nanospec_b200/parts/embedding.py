"""Token embedding into the float32 residual stream (model/llama.py:214,221: a plain row
gather, no scaling) and the output head (model/llama.py:262,286: logits = h W^T, no bias, no
soft-cap), which may share the embedding's table."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec
from .context import StepContext
from .registry import register_part


@register_part("embedding", "table")
class TokenEmbedding(Part):
    """params: vocab, hidden."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self.table: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.vocab, self.hidden))}

    def bind(self, tensors) -> None:
        self.table = tensors["weight"].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        return ops.embed(self.table, ctx.token_ids, ctx.buffer("resid", self.hidden, torch.float32))


@register_part("head", "linear")
class LinearHead(Part):
    """params: vocab, hidden, tied_to (full name of the embedding table, or None)."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.vocab, self.hidden = int(spec["vocab"]), int(spec["hidden"])
        self.tied_to = spec.params.get("tied_to")
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.vocab, self.hidden), alias=self.tied_to)}

    def bind(self, tensors) -> None:
        self.weight = tensors["weight"]

    def forward(self, h: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """h [R, hidden] compute dtype -> float32 logits [R, vocab]."""
        if out is None:
            out = torch.empty((h.shape[0], self.vocab), dtype=torch.float32, device=h.device)
        return ops.linear(h, self.weight, out)

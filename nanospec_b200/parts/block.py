"""How a layer's parts are arranged.  "prenorm" is the reference's `DecoderLayer`
(model/llama.py:198-208): x = x + mixer(norm(x)); x = x + feed_forward(norm(x)).

A block receives the float32 residual stream and a `pending` branch output that has not
been added to it yet, and returns the same pair; the sum is folded into the next norm so
that each activation is read once.

Interface of a block part:
    parts() -> dict of slot name -> Part           (for weight naming)
    forward(resid, pending, ctx, lane, writes) -> (resid, pending)
"""

from __future__ import annotations

import torch

from ..config.recipe import LayerSpec
from .context import LaneView, StepContext
from .registry import build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock:
    slots = ("norm_mixer", "mixer", "norm_feed_forward", "feed_forward")

    def __init__(self, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.layer = layer
        self.mixer = build_part("mixer", layer.mixer, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, dtype, device)
        self.norm_mixer = build_part("norm", layer.norm, dtype, device)
        self.norm_feed_forward = build_part("norm", layer.norm, dtype, device)

    def parts(self) -> dict:
        return {s: getattr(self, s) for s in self.slots}

    def forward(self, resid: torch.Tensor, pending: torch.Tensor | None, ctx: StepContext, lane: LaneView,
                writes: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
        x = self.norm_mixer.add_norm(resid, pending, ctx)
        a = self.mixer.forward(x, ctx, lane, writes)
        x = self.norm_feed_forward.add_norm(resid, a, ctx)
        return resid, self.feed_forward.forward(x, ctx)

"""How a layer's parts are arranged.  "prenorm" is the reference's `DecoderLayer`
(model/llama.py:198-208): x = x + mixer(norm(x)); x = x + feed_forward(norm(x)).

A block receives the float32 residual stream and a `pending` branch output that has not
been added to it yet, and returns the same pair; the sum is folded into the next norm so
that each activation is read once.

In a decode step of a few tokens the two norm kernels of a layer can go: when the part before a
norm can feed a sink and the part after it takes row-scaled input (`Part.feeds_norm_sink`,
`Part.takes_row_scaled`), the product before the norm adds its output to the stream and prepares the
norm's input in its epilogue, and the product after it applies the norm's scale.  `follow` is the
block that runs next (or None): its first norm is the one after this block's feed-forward.

Interface of a block part (built from a whole `LayerSpec`):
    mixer                                          the block's mixer part: the model asks it for the lane's cache and state needs
    parts() -> dict of slot name -> Part           (for weight naming: `LayerSpec.names` maps each slot to its sub-prefix)
    forward(resid, pending, ctx, lane, writes) -> (resid, pending)
    takes_follow = True                            (optional) forward() also accepts `follow=`, the block that runs next
    input_norm_sink(resid, ctx) -> ops.NormSink or None   (optional; None or absent: the block's first norm cannot be folded)
The built-in mixers and feed-forwards return their result in the step's "branch" buffer: an arrangement that needs
two branch outputs at once copies the first before it runs the second.
"""

from __future__ import annotations

import torch

from ..config.recipe import LayerSpec
from .context import LaneView, StepContext
from .registry import build_part, register_part


def _can(part, what: str, n_tokens: int) -> bool:
    """A part's optional capability (`takes_row_scaled`, `feeds_norm_sink`); parts that do not know of it have none."""
    f = getattr(part, what, None)
    return bool(f(n_tokens)) if callable(f) else False


@register_part("block", "prenorm")
class PreNormBlock:
    slots = ("norm_mixer", "mixer", "norm_feed_forward", "feed_forward")
    takes_follow = True  # forward() accepts the block that runs next

    def __init__(self, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.layer = layer
        self.mixer = build_part("mixer", layer.mixer, dtype, device)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, dtype, device)
        self.norm_mixer = build_part("norm", layer.norm, dtype, device)
        self.norm_feed_forward = build_part("norm", layer.norm, dtype, device)

    def parts(self) -> dict:
        return {s: getattr(self, s) for s in self.slots}

    def input_norm_sink(self, resid: torch.Tensor, ctx: StepContext):
        """What the product before this block needs to fold the block's first norm in, or None."""
        if _can(self.mixer, "takes_row_scaled", ctx.n_tokens) and hasattr(self.norm_mixer, "sink"):
            return self.norm_mixer.sink(resid, ctx)
        return None

    def forward(self, resid: torch.Tensor, pending, ctx: StepContext, lane: LaneView, writes: bool = True,
                follow=None) -> tuple[torch.Tensor, torch.Tensor]:
        n = ctx.n_tokens
        x = self.norm_mixer.add_norm(resid, pending, ctx)
        if _can(self.mixer, "feeds_norm_sink", n) and _can(self.feed_forward, "takes_row_scaled", n) \
                and hasattr(self.norm_feed_forward, "sink"):
            a = self.mixer.forward(x, ctx, lane, writes, sink=self.norm_feed_forward.sink(resid, ctx))
        else:
            a = self.mixer.forward(x, ctx, lane, writes)
        x = self.norm_feed_forward.add_norm(resid, a, ctx)
        sink = None
        if follow is not None and _can(self.feed_forward, "feeds_norm_sink", n) and hasattr(follow, "input_norm_sink"):
            sink = follow.input_norm_sink(resid, ctx)
        if sink is not None:
            return resid, self.feed_forward.forward(x, ctx, sink=sink)
        return resid, self.feed_forward.forward(x, ctx)

"""The dense gated feed-forward of the reference (`MLP`, model/llama.py:187-195):
down(silu(gate(x)) * up(x)), no biases.  Gate and up are one packed projection [gate | up].

Interface of a feed-forward part:
    forward(x, ctx) -> y        x, y: [N, hidden] in the compute dtype
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec
from .context import StepContext
from .registry import register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """params: hidden, intermediate."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden"])
        self.inter = int(spec["intermediate"])
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {
            "gate_proj.weight": WeightSpec((self.inter, self.hidden)),
            "up_proj.weight": WeightSpec((self.inter, self.hidden)),
            "down_proj.weight": WeightSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gu = ops.linear(x, self.w_gate_up, ctx.buffer("gate_up", 2 * self.inter))
        act = ops.swiglu(gu, ctx.buffer("ffn_act", self.inter))
        return ops.linear(act, self.w_down, ctx.buffer("branch", self.hidden))

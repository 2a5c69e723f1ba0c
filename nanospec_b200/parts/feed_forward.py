"""The dense gated feed-forward of the reference (`MLP`, model/llama.py:187-195):
down(silu(gate(x)) * up(x)), no biases.  Gate and up are one packed projection: runs of 64 gate rows
followed by the 64 matching up rows when the intermediate size is a multiple of 64 (a decode step's
product then applies the activation in its epilogue), [gate | up] otherwise.

Interface of a feed-forward part:
    forward(x, ctx) -> y        x, y: [N, hidden] in the compute dtype
and, optionally, the folding of norms into its products (`Part.takes_row_scaled`, `Part.feeds_norm_sink`).
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
        self.gate_block = 0

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {
            "gate_proj.weight": WeightSpec((self.inter, self.hidden)),
            "up_proj.weight": WeightSpec((self.inter, self.hidden)),
            "down_proj.weight": WeightSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors) -> None:
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        self.gate_block = ops.GATE_BLOCK if self.inter % ops.GATE_BLOCK == 0 else 0
        if self.gate_block:
            b = self.gate_block
            packed = torch.stack([gate.view(self.inter // b, b, self.hidden), up.view(self.inter // b, b, self.hidden)], dim=1)
            self.w_gate_up = packed.reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def takes_row_scaled(self, n_tokens: int) -> bool:
        return ops.norm_fusion_ok(n_tokens, self.dtype, self.w_gate_up)

    def feeds_norm_sink(self, n_tokens: int) -> bool:
        return ops.norm_fusion_ok(n_tokens, self.dtype, self.w_down)

    def forward(self, x, ctx: StepContext, sink: ops.NormSink | None = None):
        act = ops.gated_linear(x, self.w_gate_up, ctx.buffer("ffn_act", self.inter), ctx.buffer("gate_up", 2 * self.inter),
                               self.gate_block)
        return ops.linear(act, self.w_down, ctx.buffer("branch", self.hidden), sink=sink)

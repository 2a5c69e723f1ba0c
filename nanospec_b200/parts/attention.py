"""Grouped-query attention over the paged cache (the reference's `Attention`,
model/llama.py:161-184): packed q/k/v projection without bias, position encoding of q and
k, the step's keys and values written to their pages, softmax(q k^T / sqrt(d)) v over every
key at or before the query's position (and inside the window, if one is set), output
projection.  Query head h reads kv head h // (heads / kv_heads).

Interface of a mixer part:
    cache_need() -> CacheNeed | None      paged storage wanted per token
    state_need() -> StateNeed | None      fixed-size state wanted per request
    forward(x, ctx, lane, writes) -> y    x, y: [N, hidden] in the compute dtype
A mixer may also take part in folding the norms into its products (`Part.takes_row_scaled`,
`Part.feeds_norm_sink`); this one does.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import CacheNeed, Part, StateNeed, WeightSpec
from .context import LaneView, StepContext
from .registry import build_part, register_part


@register_part("mixer", "gqa_attention")
class GQAAttention(Part):
    """params: hidden, heads, kv_heads, head_dim, window (0 = all keys), position (PartSpec),
    scale (optional; default 1/sqrt(head_dim))."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads cannot be shared among {self.kv_heads} kv heads")
        self.q_size = self.heads * self.head_dim
        self.kv_size = self.kv_heads * self.head_dim
        self.position = build_part("position", p["position"], dtype, device) if p.get("position") is not None else None
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {
            "q_proj.weight": WeightSpec((self.q_size, self.hidden)),
            "k_proj.weight": WeightSpec((self.kv_size, self.hidden)),
            "v_proj.weight": WeightSpec((self.kv_size, self.hidden)),
            "o_proj.weight": WeightSpec((self.hidden, self.q_size)),
        }

    def bind(self, tensors) -> None:
        # one packed projection [q | k | v]: one matrix product instead of three
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()

    def cache_need(self) -> CacheNeed | None:
        return CacheNeed(self.kv_heads, self.head_dim, self.window)

    def state_need(self) -> StateNeed | None:
        return None

    def takes_row_scaled(self, n_tokens: int) -> bool:
        return ops.norm_fusion_ok(n_tokens, self.dtype, self.w_qkv)

    def feeds_norm_sink(self, n_tokens: int) -> bool:
        return ops.norm_fusion_ok(n_tokens, self.dtype, self.w_o)

    def forward(self, x, ctx: StepContext, lane: LaneView, writes: bool = True, sink: ops.NormSink | None = None):
        qkv = ctx.buffer("qkv", self.q_size + 2 * self.kv_size)
        fused = getattr(self.position, "project_rotate_store", None)
        if fused is None or not fused(x, self.w_qkv, qkv, ctx, lane, self.heads, self.kv_heads, self.head_dim, writes):
            ops.linear(x, self.w_qkv, qkv)
            if self.position is not None:
                self.position.rotate_and_store(qkv, ctx, lane, self.heads, self.kv_heads, self.head_dim, writes)
            elif writes:
                ops.kv_store(qkv, ctx, lane, self.heads, self.kv_heads, self.head_dim)
        attn = ctx.buffer("attn_out", self.q_size)
        ops.attention(qkv, lane, ctx, attn, self.heads, self.kv_heads, self.head_dim, self.scale, self.window)
        return ops.linear(attn, self.w_o, ctx.buffer("branch", self.hidden), sink=sink)

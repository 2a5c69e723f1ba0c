"""Rotary position encoding, with the llama3 wavelength-banded frequency rescale.

The frequencies are computed once, in float32, with the reference's expressions in the
reference's order (model/llama.py:98-118); the kernel forms angle = float(position) *
inv_freq[j] in float32 and rotates the pairs (j, j + head_dim/2) ("rotate half",
model/llama.py:150-158).

Interface of a position part used by an attention mixer:
    rotate_and_store(qkv, ctx, lane, nq, nkv, head_dim, writes)
        rotates q and k inside the packed projection [q | k | v]; when `writes`, stores the
        rotated k and v at each token's slot of `lane`.
    project_rotate_store(x, w_qkv, qkv, ctx, lane, nq, nkv, head_dim, writes) -> bool      (optional)
        the projection itself with the rotation and the store in its epilogue; False (nothing done)
        when the step does not fit, and the mixer then runs the projection and `rotate_and_store`.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import Part
from .context import LaneView, StepContext
from .registry import register_part


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """float32 [head_dim / 2] on the CPU; `scaling` holds the llama3 block or is None."""
    ar = torch.arange(0, head_dim, 2, dtype=torch.int64).float()
    inv_freq = 1.0 / (theta ** (ar / head_dim))
    if scaling is None:
        return inv_freq
    factor = scaling["factor"]
    low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
    old_len = scaling["original_max_position_embeddings"]
    low_wavelen, high_wavelen = old_len / low, old_len / high
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old_len / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) * ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, scaled)


@register_part("position", "rope")
class RotaryEncoding(Part):
    """params: head_dim, theta, scaling (None or the llama3 block as a dict)."""

    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.head_dim = int(spec["head_dim"])
        scaling = spec.params.get("scaling")
        self.inv_freq_host = rope_inverse_frequencies(self.head_dim, float(spec["theta"]),
                                                      dict(scaling) if scaling else None)
        self._inv_freq: torch.Tensor | None = None

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            self._inv_freq = self.inv_freq_host.to(self.device).contiguous()
        return self._inv_freq

    def rotate_and_store(self, qkv: torch.Tensor, ctx: StepContext, lane: LaneView, nq: int, nkv: int,
                         head_dim: int, writes: bool) -> None:
        ops.rope_kv_write(qkv, ctx.positions, ctx.token_req, lane.block_table, self.inv_freq, lane.k, lane.v,
                          lane.page_size, nq, nkv, head_dim, write_kv=writes)

    def project_rotate_store(self, x, w_qkv: torch.Tensor, qkv: torch.Tensor, ctx: StepContext, lane: LaneView, nq: int,
                             nkv: int, head_dim: int, writes: bool) -> bool:
        return ops.linear_rope(x, w_qkv, qkv, ctx.positions, ctx.token_req, lane.block_table, self.inv_freq, lane.k, lane.v,
                               lane.page_size, nq, nkv, head_dim, write_kv=writes)

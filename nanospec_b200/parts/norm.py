"""RMSNorm over the float32 residual stream, fused with the residual sum.

Formula of the reference (model/llama.py:86-95): h = x * rsqrt(mean(x^2) + eps), y = gain * h,
eps inside the root, the gain applied as is (not 1 + gain).  Here the statistics, the scale
and the gain product are all float32 and the result is rounded once to the compute dtype.

Interface of a norm part:
    add_norm(resid, pending, ctx, rows=None, out_name="normed") -> normed
        resid    [N, H] float32, updated in place with `pending` when that is given
        pending  [N, H] compute dtype or None: a branch output not yet added to the stream
        rows     int32 device tensor or None: only these rows are produced (resid untouched)
        out_name the step buffer (`ctx.buffer(out_name, H, rows=...)`) that takes the result
    sink(resid, ctx) -> ops.NormSink    (optional) what a product needs to fold this norm and the sum
                                        before it into its epilogue; `add_norm` hands the product's
                                        `ops.RowScaled` result on unchanged.  A norm without `sink`
                                        is never folded.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec
from .context import StepContext
from .registry import register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    def __init__(self, spec, dtype, device) -> None:
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden"])
        self.eps = float(spec["eps"])
        self.gain: torch.Tensor | None = None

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.hidden,), rule="float32", init="gain")}

    def bind(self, tensors) -> None:
        self.gain = tensors["weight"].contiguous()

    def sink(self, resid: torch.Tensor, ctx: StepContext) -> ops.NormSink:
        return ops.NormSink(resid, self.gain, self.eps, ctx.workspace)

    def add_norm(self, resid: torch.Tensor, pending, ctx: StepContext,
                 rows: torch.Tensor | None = None, out_name: str = "normed"):
        if isinstance(pending, ops.RowScaled):
            # a product has added its output to the stream and prepared this norm's input already
            if pending.gain is not self.gain or rows is not None:
                raise ValueError("a RowScaled reached a norm it was not made for")
            return pending
        n = resid.shape[0] if rows is None else rows.numel()
        out = ctx.buffer(out_name, self.hidden, rows=n)
        return ops.add_rmsnorm(resid, pending, self.gain, self.eps, out, rows=rows)

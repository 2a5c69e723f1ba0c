"""A decoder assembled from a `ModelRecipe`: embedding, blocks run in the recipe's order on
the recipe's cache lanes, final norm at the wanted rows, head.  The reference's counterpart
is `LlamaModel` / `LlamaForCausalLM` (model/llama.py:211-286); here nothing is specific to
one architecture."""

from __future__ import annotations

import torch

from ..config.recipe import ModelRecipe
from .base import CacheNeed, StateNeed, WeightSpec
from .context import StepContext
from .registry import build_block, build_part


class DecoderModel:
    def __init__(self, recipe: ModelRecipe, dtype: torch.dtype, device: torch.device | str) -> None:
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        self.recipe = recipe
        self.dtype = dtype
        self.device = torch.device(device)
        self.embedding = build_part("embedding", recipe.embedding, dtype, self.device)
        self.blocks = [build_block(layer, dtype, self.device) for layer in recipe.layers]
        self.final_norm = build_part("norm", recipe.final_norm, dtype, self.device)
        self.head = build_part("head", recipe.head, dtype, self.device)
        self.vocab_size = recipe.vocab_size
        self.hidden_size = recipe.hidden_size
        self.bound = False

    # ---- weights ---------------------------------------------------------------------
    def _named_parts(self):
        r = self.recipe
        yield r.embedding.params.get("name", "model.embed_tokens") + ".", self.embedding
        for layer, block in zip(r.layers, self.blocks):
            for slot, part in block.parts().items():
                yield layer.prefix + layer.names[slot], part
        yield r.final_norm_prefix, self.final_norm
        yield r.head.params.get("name", "lm_head") + ".", self.head

    def weight_specs(self) -> dict[str, WeightSpec]:
        """Full checkpoint name -> what is wanted under it."""
        out: dict[str, WeightSpec] = {}
        for prefix, part in self._named_parts():
            for name, spec in part.weight_specs().items():
                out[prefix + name] = spec
        return out

    def bind(self, weights: dict[str, torch.Tensor]) -> None:
        """`weights`: full name -> tensor on the device, already cast (see weights/loader.py)."""
        for prefix, part in self._named_parts():
            part.bind({name: weights[prefix + name] for name in part.weight_specs()})
        self.bound = True

    # ---- cache needs, one entry per lane ------------------------------------------------
    def lane_needs(self) -> list[tuple[CacheNeed | None, StateNeed | None]]:
        needs: dict[int, tuple[CacheNeed | None, StateNeed | None]] = {}
        for run in self.recipe.order:
            if run.writes:
                mixer = self.blocks[run.layer].mixer
                needs[run.lane] = (mixer.cache_need(), mixer.state_need())
        return [needs[i] for i in range(len(needs))]

    # ---- one step ----------------------------------------------------------------------
    def forward(self, ctx: StepContext, want_rows: torch.Tensor | None, all_rows: bool = False) -> torch.Tensor | None:
        """Runs the step's tokens through every block (which fills the cache).  Returns the
        normed hidden states of `want_rows` (int32 device tensor of row numbers), of every row
        when `all_rows`, or None when nothing is wanted."""
        resid = self.embedding.forward(ctx)
        pending = None
        order = self.recipe.order
        for i, run in enumerate(order):
            # the block that runs next: its first norm may be folded into this block's last product
            follow = self.blocks[order[i + 1].layer] if i + 1 < len(order) else None
            block = self.blocks[run.layer]
            if follow is not None and getattr(block, "takes_follow", False):
                resid, pending = block.forward(resid, pending, ctx, ctx.lanes[run.lane], run.writes, follow=follow)
            else:
                resid, pending = block.forward(resid, pending, ctx, ctx.lanes[run.lane], run.writes)
        if want_rows is None and not all_rows:
            return None
        return self.final_norm.add_norm(resid, pending, ctx, rows=want_rows, out_name="final_normed")

    def logits(self, hidden: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        return self.head.forward(hidden, out)

"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

A step may hold portions of prompts beside single decoded tokens, cut anywhere.  It runs
only the tokens it is given, as one flattened batch, on the cache that earlier steps left:
one forward pass for everything, where the reference runs one pass for the decoding
requests and another for the newly admitted prompts (engine/engine.py:226-229).  The batch
description follows the reference's `AttnMeta.from_rows` (kv/cache.py:113-157) - positions
per token, a block table per request - except that cache slots are computed on the device
from the block table instead of being uploaded per token.

`ModelRunner` owns the model, the cache manager with its device storage, and the scratch
buffers; generation (engine.py) and trace replay (bin/trace_run) both drive this one object.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops
from ..cache import CacheManager, CacheStorage
from ..parts.context import StepContext, Workspace
from ..parts.model import DecoderModel


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places (indices into
    `tokens`) whose logits are wanted."""

    req_id: int
    tokens: list[int]
    want: list[int] = field(default_factory=list)


class _Staging:
    """Pinned host buffers for the step description, used in turn so that the host never
    overwrites one that a copy may still be reading."""

    def __init__(self, depth: int = 2) -> None:
        self.bufs: list[torch.Tensor | None] = [None] * depth
        self.events: list[torch.cuda.Event | None] = [None] * depth
        self.turn = 0

    def get(self, n_ints: int) -> tuple[torch.Tensor, int]:
        i = self.turn
        self.turn = (self.turn + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.bufs[i]
        if buf is None or buf.numel() < n_ints:
            buf = torch.empty(max(n_ints, 4096), dtype=torch.int32).pin_memory()
            self.bufs[i] = buf
        return buf, i

    def replace(self, i: int, n_ints: int) -> torch.Tensor:
        """A larger buffer in place of buffer `i`, which the caller holds and no copy reads."""
        self.bufs[i] = torch.empty(n_ints, dtype=torch.int32).pin_memory()
        return self.bufs[i]

    def mark(self, i: int) -> None:
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class ModelRunner:
    def __init__(self, model: DecoderModel, num_blocks: int, block_size: int, max_requests: int) -> None:
        if not model.bound:
            raise RuntimeError("the model has no weights bound")
        if model.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device; there is no CPU path")
        self.model = model
        self.device, self.dtype = model.device, model.dtype
        needs = model.lane_needs()
        self.manager = CacheManager(needs, num_blocks, block_size, max_requests)
        self.storage = CacheStorage(self.manager, needs, self.dtype, self.device)
        self.workspace = Workspace(self.device)
        self.block_size = block_size
        self.max_positions = model.recipe.max_positions
        self._staging = _Staging()
        self._staging_ints = 1 << 16
        self._meta_dev: torch.Tensor | None = None
        self.h2d_bytes_last = 0

    # ---- request life -------------------------------------------------------------------
    def begin(self, req_id: int) -> None:
        self.manager.begin(req_id)

    def end(self, req_id: int) -> None:
        self.manager.end(req_id)

    # ---- building the batch ----------------------------------------------------------------
    def build_context(self, entries: list[StepEntry], take: tuple[list[int], torch.Tensor, list[int]] | None = None,
                      extra: np.ndarray | None = None) -> tuple[StepContext, torch.Tensor | None, int]:
        """Reserves pages (for every entry, or for none: `PoolExhausted` and `ValueError` leave the cache as it
        was), lays the step description out in one pinned buffer - in native code, from the block tables that
        live there - and copies it to the device once.  Returns (context, wanted rows on the device or None, n wanted).
        `take` = (token rows of this step, an int32 device tensor, rows of it): those token ids are not
        known to the host yet and are taken from the tensor on the device (the entries carry a placeholder).
        `extra`: int32 values that travel with the description (`ctx.extras["extra"]` is their place on the device):
        everything a step needs from the host goes in this one copy from pinned memory, since a copy from ordinary
        memory would make the host wait for all the work queued before it."""
        m = self.manager
        B = len(entries)
        req_ids = np.fromiter((e.req_id for e in entries), dtype=np.int64, count=B)
        if len(set(req_ids.tolist())) != B:
            raise ValueError("a request may appear once in a step")
        q_lens = [len(e.tokens) for e in entries]
        N = sum(q_lens)
        ids_np = np.empty(max(N, 1), dtype=np.int32)
        want_rows: list[int] = []
        at = 0
        for e, n in zip(entries, q_lens):
            if n == 0:
                raise ValueError(f"request {e.req_id} brings no tokens to the step")
            if n == 1:
                ids_np[at] = e.tokens[0]
            else:
                ids_np[at: at + n] = e.tokens
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.req_id} wants logits at place {w} of {n} tokens")
                want_rows.append(at + w)
            at += n
        vocab = self.model.vocab_size
        if N and (ids_np[:N].min() < 0 or ids_np[:N].max() >= vocab):
            bad = int(ids_np[:N][(ids_np[:N] < 0) | (ids_np[:N] >= vocab)][0])
            raise ValueError(f"token id {bad} is outside the vocabulary of {vocab}")
        q_lens_np = np.asarray(q_lens, dtype=np.int32)
        want_np = np.asarray(want_rows, dtype=np.int32)
        take_dst = np.asarray(take[0] if take else [], dtype=np.int32)
        take_src = np.asarray(take[2] if take else [], dtype=np.int32)
        extra_np = np.zeros(0, dtype=np.int32) if extra is None else np.ascontiguousarray(extra, dtype=np.int32)
        host, turn = self._staging.get(self._staging_ints)
        while True:
            try:
                offsets, widths, counts, total, max_q, max_kv = m.pack_step(
                    req_ids, q_lens_np, ids_np, want_np, take_dst, take_src, extra_np, (ops.TILE_Q, ops.TILE_Q_TCGEN05),
                    self.max_positions, host.numpy(), host.numel())
                break
            except BufferError as need:  # the description is larger than any before: a larger pinned buffer, once
                self._staging_ints = 2 * int(need.args[0])
                host = self._staging.replace(turn, self._staging_ints)
        if self._meta_dev is None or self._meta_dev.numel() < total:
            self._meta_dev = torch.empty(max(2 * total, 4096), dtype=torch.int32, device=self.device)
        dev = self._meta_dev
        dev[:total].copy_(host[:total], non_blocking=True)
        self._staging.mark(turn)
        self.h2d_bytes_last = total * 4

        def view(i: int, n: int) -> torch.Tensor:
            return dev[offsets[i]: offsets[i] + n]

        if len(take_dst):
            ops.take_ids(view(0, N), view(7, len(take_dst)), take[1], view(8, len(take_src)))
        group_tables = [view(14 + gi, B * widths[gi]).view(B, widths[gi]) for gi in range(len(m.groups))]
        self.storage.zero_state_slots(m.take_fresh_slots())
        host_np = host.numpy()
        kv_lens = host_np[offsets[4]: offsets[4] + B].tolist()
        ctx = StepContext(
            n_tokens=N, n_requests=B,
            token_ids=view(0, N), positions=view(1, N), token_req=view(2, N), qo_indptr=view(3, B + 1),
            kv_len=view(4, B), state_slot=view(5, B),
            q_lens=q_lens, kv_lens=kv_lens,
            lanes=self.storage.lane_views(group_tables),
            workspace=self.workspace, dtype=self.dtype, device=self.device,
            max_q_len=max_q, max_kv_len=max_kv, state_slots_host=host_np[offsets[5]: offsets[5] + B].tolist(),
        )
        ctx.extras["req_ids"] = req_ids
        ctx.extras["extra"] = view(12, len(extra_np))
        # which token rows decode and the query tiles of the prompt portions (ops.attention reads this)
        n_decode, n_a, n_b, max_kv_decode, n_work, work_slots = counts
        ctx.extras["attention_plan"] = {
            "n_decode": n_decode,
            "decode_rows": None if n_decode == N or not n_decode else view(9, n_decode),
            "tiles": view(10, 2 * n_a).view(n_a, 2) if n_a else None,
            "tiles_tc": view(11, 2 * n_b).view(n_b, 2) if n_b else None,
            "max_kv_len": max_kv_decode or None,
            # the decode kernel's work list (a request much longer than the others comes in parts) and the slots of
            # scratch that its parts need
            "work": view(13, 4 * n_work) if n_work else None, "work_slots": work_slots,
        }
        n_want = len(want_rows)
        return ctx, (view(6, n_want) if n_want else None), n_want

    # ---- running ------------------------------------------------------------------------
    def run(self, entries: list[StepEntry], take=None) -> torch.Tensor | None:
        """Runs the step and returns the normed hidden states at the wanted places, in the
        order of the entries and of their `want` lists ([n_wanted, hidden]), or None.
        `take`: token ids that are still on the device (see build_context)."""
        ctx, want_rows, n_want = self.build_context(entries, take)
        return self.forward(ctx, want_rows)

    def forward(self, ctx: StepContext, want_rows: torch.Tensor | None) -> torch.Tensor | None:
        """The model over a context that `build_context` made, then the pages that windows have passed go back."""
        hidden = self.model.forward(ctx, want_rows)  # None when nothing is wanted: the blocks still fill the cache
        self.manager.trim_many(ctx.extras["req_ids"])
        return hidden

    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """run() followed by the head: float32 logits [n_wanted, vocab] (None if nothing is wanted)."""
        hidden = self.run(entries)
        return None if hidden is None else self.model.logits(hidden)

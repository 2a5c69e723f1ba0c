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
from ..cache import CacheManager, CacheStorage, PoolExhausted
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
        self._meta_dev: torch.Tensor | None = None
        self.h2d_bytes_last = 0

    # ---- request life -------------------------------------------------------------------
    def begin(self, req_id: int) -> None:
        self.manager.begin(req_id)

    def end(self, req_id: int) -> None:
        self.manager.end(req_id)

    # ---- building the batch ----------------------------------------------------------------
    def _reserve(self, entries: list[StepEntry]) -> None:
        done: list[tuple[int, int]] = []
        try:
            for e in entries:
                if not e.tokens:
                    raise ValueError(f"request {e.req_id} brings no tokens to the step")
                if self.manager.seq_len[e.req_id] + len(e.tokens) > self.max_positions:
                    raise ValueError(
                        f"request {e.req_id} would reach {self.manager.seq_len[e.req_id] + len(e.tokens)} positions; "
                        f"the model's limit is {self.max_positions}")
                before = self.manager.seq_len[e.req_id]
                self.manager.extend(e.req_id, len(e.tokens))
                done.append((e.req_id, before))
        except (PoolExhausted, ValueError):
            for rid, before in reversed(done):
                self.manager.rollback(rid, before)
            raise

    def build_context(self, entries: list[StepEntry], take: tuple[list[int], torch.Tensor, list[int]] | None = None,
                      ) -> tuple[StepContext, torch.Tensor | None, int]:
        """Reserves pages, lays the step description out in one pinned buffer and copies it
        to the device once.  Returns (context, wanted rows on the device or None, n wanted).
        `take` = (token rows of this step, an int32 device tensor, rows of it): those token ids are not
        known to the host yet and are taken from the tensor on the device (the entries carry a placeholder)."""
        ids = [e.req_id for e in entries]
        if len(set(ids)) != len(ids):
            raise ValueError("a request may appear once in a step")
        vocab = self.model.vocab_size
        m = self.manager
        B = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        N = sum(q_lens)
        ids_np = np.empty(N, dtype=np.int64)
        at = 0
        for e, n in zip(entries, q_lens):
            if n == 1:
                ids_np[at] = e.tokens[0]
            else:
                ids_np[at: at + n] = e.tokens
            at += n
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.req_id} wants logits at place {w} of {n} tokens")
        if N and (ids_np.min() < 0 or ids_np.max() >= vocab):
            bad = int(ids_np[(ids_np < 0) | (ids_np >= vocab)][0])
            raise ValueError(f"token id {bad} is outside the vocabulary of {vocab}")
        starts = [m.seq_len[e.req_id] for e in entries]
        self._reserve(entries)

        kv_lens = [s + n for s, n in zip(starts, q_lens)]
        q_lens_np = np.asarray(q_lens, dtype=np.int32)
        qo_indptr = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(q_lens_np, out=qo_indptr[1:])
        token_req = np.repeat(np.arange(B, dtype=np.int32), q_lens_np)
        # token i of request b sits at position starts[b] + (i - qo_indptr[b])
        positions = np.arange(N, dtype=np.int32) + np.repeat(np.asarray(starts, dtype=np.int32) - qo_indptr[:-1], q_lens_np)
        want_rows = [int(qo_indptr[b]) + w for b, e in enumerate(entries) for w in e.want]
        slots = [m.state_slot(e.req_id) for e in entries]
        tables, widths = [], []
        for gi in range(len(m.groups)):
            rows = [m.table(gi, e.req_id) for e in entries]
            width = max(1, max(len(r) for r in rows))
            table = np.zeros((B, width), dtype=np.int32)
            for b, r in enumerate(rows):
                table[b, : len(r)] = r
            tables.append(table.reshape(-1))
            widths.append(width)

        take_dst = np.asarray(take[0] if take else [], dtype=np.int32)
        take_src = np.asarray(take[2] if take else [], dtype=np.int32)
        parts = [ids_np.astype(np.int32), positions, token_req, qo_indptr, np.asarray(kv_lens, dtype=np.int32),
                 np.asarray(slots, dtype=np.int32), np.asarray(want_rows, dtype=np.int32), take_dst, take_src, *tables]
        offsets, total = [], 0
        for p in parts:
            offsets.append(total)
            total += len(p) + (-len(p) % 4)  # 16-byte aligned sections
        host, turn = self._staging.get(total)
        host_np = host.numpy()
        for off, p in zip(offsets, parts):
            host_np[off: off + len(p)] = p
        if self._meta_dev is None or self._meta_dev.numel() < total:
            self._meta_dev = torch.empty(max(total, 4096), dtype=torch.int32, device=self.device)
        dev = self._meta_dev
        dev[:total].copy_(host[:total], non_blocking=True)
        self._staging.mark(turn)
        self.h2d_bytes_last = total * 4

        def view(i: int, n: int) -> torch.Tensor:
            return dev[offsets[i]: offsets[i] + n]

        if take and len(take_dst):
            ops.take_ids(view(0, N), view(7, len(take_dst)), take[1], view(8, len(take_src)))
        group_tables = [view(9 + gi, B * widths[gi]).view(B, widths[gi]) for gi in range(len(m.groups))]
        self.storage.zero_state_slots(m.take_fresh_slots())
        ctx = StepContext(
            n_tokens=N, n_requests=B,
            token_ids=view(0, N), positions=view(1, N), token_req=view(2, N), qo_indptr=view(3, B + 1),
            kv_len=view(4, B), state_slot=view(5, B),
            q_lens=q_lens, kv_lens=kv_lens,
            lanes=self.storage.lane_views(group_tables),
            workspace=self.workspace, dtype=self.dtype, device=self.device,
            max_q_len=max(q_lens), max_kv_len=max(kv_lens), state_slots_host=slots,
        )
        n_want = len(want_rows)
        return ctx, (view(6, n_want) if n_want else None), n_want

    # ---- running ------------------------------------------------------------------------
    def run(self, entries: list[StepEntry], take=None) -> torch.Tensor | None:
        """Runs the step and returns the normed hidden states at the wanted places, in the
        order of the entries and of their `want` lists ([n_wanted, hidden]), or None.
        `take`: token ids that are still on the device (see build_context)."""
        ctx, want_rows, n_want = self.build_context(entries, take)
        hidden = self.model.forward(ctx, want_rows)  # None when nothing is wanted: the blocks still fill the cache
        for e in entries:
            self.manager.trim(e.req_id)
        return hidden

    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """run() followed by the head: float32 logits [n_wanted, vocab] (None if nothing is wanted)."""
        hidden = self.run(entries)
        return None if hidden is None else self.model.logits(hidden)

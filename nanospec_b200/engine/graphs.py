"""CUDA-graph replay of decode-only steps, one graph per batch bucket.

As in the reference (engine/graphs.py:22,109-113,171-210) a step in which every request
brings exactly one token is padded up to the next bucket of (1, 2, 4, ..., 64) requests and
replayed from a graph captured once for that bucket.  Differences: the attention kernels
read sequence lengths and block tables from device memory, so nothing has to be planned on
the host outside the graph; padding rows carry request index -1 and are skipped by every
kernel instead of writing to a reserved page; and the head projection and the sampling
kernel are part of the graph, so one replay goes from token ids to next tokens.

The step description of a bucket lives in one pinned host buffer that is copied to one
device buffer per step; the graph's kernels hold pointers into that device buffer.
"""

from __future__ import annotations

import ctypes
import dataclasses

import numpy as np
import torch

from .. import ops
from ..parts.context import StepContext, Workspace
from .scheduler import Scheduled
from .step import ModelRunner, StepEntry


def _pad4(n: int) -> int:
    return n + (-n % 4)


class _Bucket:
    """Static buffers and the captured graph of one batch size."""

    def __init__(self, runner: ModelRunner, size: int, table_width: int, pool) -> None:
        self.size, self.width = size, table_width
        self.scratch_slot = runner.manager.scratch_slot  # where padding rows keep their (meaningless) state
        # scratch of this bucket alone: the graph holds pointers into it, so nothing else may ever make it grow
        workspace = self.workspace = Workspace(runner.device)
        m = runner.manager
        n_groups = len(m.groups)
        names = ["positions", "token_req", "qo_indptr", "kv_len", "slots", "want_rows", "top_k",
                 "temperature", "top_p", "u", "take_dst", "take_src", "work"]
        # the decode attention kernel's work list: a request whose context is much longer than the others' comes in parts,
        # each an item of its own; the bucket has room for this many items beyond its rows
        self.n_work = size + min(size, 16)
        self.off: dict[str, int] = {}
        total = 0
        for nm in names:
            self.off[nm] = total
            total += _pad4(4 * self.n_work if nm == "work" else size + 1 if nm == "qo_indptr" else size)
        self.table_off = []
        for _ in range(n_groups):
            self.table_off.append(total)
            total += _pad4(size * table_width)
        self.total = total
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.host_f32 = self.host.view(torch.float32).numpy()
        self.dev = torch.zeros(total, dtype=torch.int32, device=runner.device)
        # token ids live apart from the rest: a step launched ahead of its predecessor's results takes
        # them on the device, from the predecessor's sampled tokens (`out_token` of a bucket, or an eager step's)
        self.ids_host = torch.full((size,), -1, dtype=torch.int32).pin_memory()
        self.ids_dev = torch.full((size,), -1, dtype=torch.int32, device=runner.device)
        self.table_off_c = (ctypes.c_int * max(n_groups, 1))(*self.table_off)
        self.copied = torch.cuda.Event()
        self.out_token = torch.zeros(size, dtype=torch.int32, device=runner.device)
        self.out_lp = torch.zeros(2, size, dtype=torch.float32, device=runner.device)
        # results on the host, two sets used in turn.  They are copied whole: a copy of part of each row is not
        # contiguous, and such a copy between device and host goes through a temporary and blocks the host
        self.tok_host = [torch.zeros(size, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.lp_host = [torch.zeros(2, size, dtype=torch.float32).pin_memory() for _ in range(2)]
        self.out_done = [torch.cuda.Event(), torch.cuda.Event()]
        self.turn = 0
        self.logits = torch.zeros(size, runner.model.vocab_size, dtype=torch.float32, device=runner.device)
        self.sample_scratch = torch.zeros(size * 48, dtype=torch.float32, device=runner.device)
        self.graph: torch.cuda.CUDAGraph | None = None
        # fixed parts of the description
        self.host_np[self.off["qo_indptr"]: self.off["qo_indptr"] + size + 1] = np.arange(size + 1, dtype=np.int32)
        self.host_np[self.off["want_rows"]: self.off["want_rows"] + size] = np.arange(size, dtype=np.int32)
        self.host_np[self.off["work"]: self.off["work"] + 4 * self.n_work] = np.tile(np.array([-1, -1, 0, -1], dtype=np.int32), self.n_work)
        self._fill_padding(0, description=True)
        self.dev.copy_(self.host)

        def view(name: str, n: int, dtype=torch.int32) -> torch.Tensor:
            t = self.dev[self.off[name]: self.off[name] + n]
            return t if dtype == torch.int32 else t.view(dtype)

        tables = [self.dev[o: o + size * table_width].view(size, table_width) for o in self.table_off]
        self.ctx = StepContext(
            n_tokens=size, n_requests=size,
            token_ids=self.ids_dev, positions=view("positions", size), token_req=view("token_req", size),
            qo_indptr=view("qo_indptr", size + 1), kv_len=view("kv_len", size), state_slot=view("slots", size),
            q_lens=[1] * size, kv_lens=[table_width * runner.block_size] * size,
            lanes=runner.storage.lane_views(tables), workspace=workspace, dtype=runner.dtype, device=runner.device,
            max_q_len=1, max_kv_len=table_width * runner.block_size,
        )
        self.ctx.extras["graph"] = True
        # Two graphs per bucket.  The usual one runs the decode attention kernel over the first `size` items of the work list
        # (the rows, longest context first).  When some request's context is so much longer than the others' that the
        # packer has cut it into parts, the list is longer than the bucket, and a second graph, captured when that
        # first happens, runs the kernel over all `n_work` items (the unused ones cost a little, which is why the
        # usual graph does without them).
        plan = {"decode_rows": None, "n_decode": size, "tiles": None, "tiles_tc": None, "max_kv_len": None,
                "work": view("work", 4 * size), "work_slots": 2 * (self.n_work - size)}
        self.ctx.extras["attention_plan"] = plan
        self.ctx_parts = dataclasses.replace(self.ctx, extras=dict(self.ctx.extras, attention_plan=dict(plan, work=view("work", 4 * self.n_work))))
        self.want_rows = view("want_rows", size)
        self.sampling = (view("temperature", size, torch.float32), view("top_k", size), view("top_p", size, torch.float32),
                         view("u", size, torch.float32))
        self.blank = self.dev.clone()  # the description of a step of nothing but padding rows: what a capture runs on
        self.graph_parts: torch.cuda.CUDAGraph | None = None
        self.graph = self._capture(runner, pool, self.ctx)

    def _fill_padding(self, first: int, description: bool = False) -> None:
        """Sampling options and token ids of the rows from `first` on; with `description` also their request (-1),
        position, length and state slot, which a launch leaves to the cache manager's native side."""
        o, n = self.off, self.size
        self.ids_host[first:] = -1
        if description:
            self.host_np[o["token_req"] + first: o["token_req"] + n] = -1
            self.host_np[o["positions"] + first: o["positions"] + n] = 0
            self.host_np[o["kv_len"] + first: o["kv_len"] + n] = 0
            self.host_np[o["slots"] + first: o["slots"] + n] = self.scratch_slot
        self.host_np[o["top_k"] + first: o["top_k"] + n] = 0
        self.host_f32[o["temperature"] + first: o["temperature"] + n] = 0.0
        self.host_f32[o["top_p"] + first: o["top_p"] + n] = 1.0
        self.host_f32[o["u"] + first: o["u"] + n] = 0.0

    def graph_for(self, runner: ModelRunner, pool, parts: bool) -> torch.cuda.CUDAGraph:
        """The graph to replay: the usual one, or the one whose attention kernel takes the whole work list (captured at its
        first use, on a description of padding rows, before the step's own description is copied in)."""
        if not parts:
            return self.graph
        if self.graph_parts is None:
            self.dev.copy_(self.blank)
            self.ids_dev.fill_(-1)
            self.graph_parts = self._capture(runner, pool, self.ctx_parts)
        return self.graph_parts

    def _forward(self, runner: ModelRunner, ctx: StepContext) -> None:
        hidden = runner.model.forward(ctx, self.want_rows)
        z = runner.model.logits(hidden, self.logits)
        t, k, p, u = self.sampling
        ops.sample_rows(z, t, k, p, u, out=(self.out_token, self.out_lp[0], self.out_lp[1]), scratch=self.sample_scratch)

    def _capture(self, runner: ModelRunner, pool, ctx: StepContext) -> torch.cuda.CUDAGraph:
        # two eager runs on a side stream first (every row is padding, nothing touches the cache),
        # so that scratch buffers and library workspaces exist before the capture
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._forward(runner, ctx)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..ops import lib

        g = torch.cuda.CUDAGraph()
        before = lib.launch_count()
        with torch.cuda.graph(g, pool=pool):
            self._forward(runner, ctx)
        self.kernels = lib.launch_count() - before  # this framework's kernels in one replay
        self.workspace.frozen = True  # a buffer that would have to move now raises instead
        return g


class DecodeGraphs:
    def __init__(self, runner: ModelRunner, buckets=(1, 2, 4, 8, 16, 32, 64, 128, 256), record_logits: bool = False) -> None:
        self.runner = runner
        self.record_logits = record_logits
        self.sizes = tuple(sorted(buckets))
        max_context = min(runner.max_positions, runner.manager.num_blocks * runner.block_size)
        self.table_width = max(1, -(-max_context // runner.block_size))
        self.pool = torch.cuda.graph_pool_handle()
        self.buckets: dict[int, _Bucket] = {}
        self.replays = 0
        self.timing: list | None = None  # set to a list to collect (start, end) CUDA events of each replay

    def bucket_size(self, n: int) -> int | None:
        return next((b for b in self.sizes if b >= n), None)

    def can_run(self, batch: list[Scheduled]) -> bool:
        return (all(len(s.tokens) == 1 and s.samples for s in batch) and self.bucket_size(len(batch)) is not None)

    def capture_all(self, max_batch: int | None = None) -> None:
        """Captures every bucket that a batch of up to `max_batch` requests can fall into."""
        top = self.sizes[-1] if max_batch is None else (self.bucket_size(max_batch) or self.sizes[-1])
        for b in reversed(self.sizes):  # largest first: the shared pool is sized by the biggest
            if b <= top:
                self._bucket(b)

    def _bucket(self, size: int) -> _Bucket:
        if size not in self.buckets:
            self.buckets[size] = _Bucket(self.runner, size, self.table_width, self.pool)
        return self.buckets[size]

    def run(self, batch: list[Scheduled], uniforms: list[float]):
        """launch() and collect() in one: (tokens, raw log-probs, processed log-probs, logits rows or None)."""
        return self.collect(self.launch(batch, uniforms))

    def launch(self, batch: list[Scheduled], uniforms: list[float], take: tuple[torch.Tensor, list[int]] | None = None,
               ) -> "InFlight":
        """Reserves pages, fills the bucket's description, copies it and replays the graph; does not
        wait.  With `take` = (int32 device tensor, one row of it per request, or None for a request whose token the
        host knows) the step's token ids are tokens that an earlier step sampled and that the host has not seen: the
        step can be launched before they have reached it."""
        runner = self.runner
        m = runner.manager
        B = len(batch)
        bk = self._bucket(self.bucket_size(B))
        req_ids = np.fromiter((s.req.id for s in batch), dtype=np.int64, count=B)
        bk.copied.synchronize()  # the previous copy out of the pinned buffers has finished
        o, hn, hf = bk.off, bk.host_np, bk.host_f32
        # pages for one more position of every request (all or none), then positions, lengths, state slots, padding
        # rows and every group's block-table rows, written by the cache manager's native side
        m.pack_decode(req_ids, bk.size, runner.max_positions, hn, o, bk.table_off_c, bk.width, bk.n_work)
        hn[o["top_k"]: o["top_k"] + B] = [s.req.params.top_k for s in batch]
        hf[o["temperature"]: o["temperature"] + B] = [s.req.params.temperature for s in batch]
        hf[o["top_p"]: o["top_p"] + B] = [s.req.params.top_p for s in batch]
        hf[o["u"]: o["u"] + B] = uniforms
        bk._fill_padding(B)
        # has the packer cut some request's keys into parts?  (meta of an item: -1 for a whole request)
        w0 = o["work"]
        graph = bk.graph_for(runner, self.pool, bool((hn[w0 + 3: w0 + 4 * bk.n_work: 4] >= 0).any()))
        t0 = t1 = None
        if self.timing is not None:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
        n_take = 0
        if take is not None:
            # rows whose token an earlier step sampled and the host has not seen take it on the device; the others
            # (a prompt's last token, known all along) bring theirs from the host
            rows = [i for i, r in enumerate(take[1]) if r is not None]
            n_take = len(rows)
            bk.ids_host[:B] = torch.tensor([0 if take[1][i] is not None else s.tokens[0] for i, s in enumerate(batch)], dtype=torch.int32)
            hn[o["take_dst"]: o["take_dst"] + n_take] = rows
            hn[o["take_src"]: o["take_src"] + n_take] = [take[1][i] for i in rows]
        else:
            bk.ids_host[:B] = torch.tensor([s.tokens[0] for s in batch], dtype=torch.int32)
        bk.ids_dev.copy_(bk.ids_host, non_blocking=True)  # padding rows carry -1
        bk.dev.copy_(bk.host, non_blocking=True)
        bk.copied.record()
        if n_take:
            ops.take_ids(bk.ids_dev, bk.dev[o["take_dst"]: o["take_dst"] + n_take], take[0],
                         bk.dev[o["take_src"]: o["take_src"] + n_take])
        runner.h2d_bytes_last = (bk.total + bk.size) * 4
        runner.storage.zero_state_slots(m.take_fresh_slots())
        graph.replay()
        self.replays += 1
        turn = bk.turn
        bk.turn ^= 1
        bk.tok_host[turn].copy_(bk.out_token, non_blocking=True)
        bk.lp_host[turn].copy_(bk.out_lp, non_blocking=True)
        raw = bk.logits[:B].cpu() if self.record_logits else None
        bk.out_done[turn].record()
        if t1 is not None:
            t1.record()
            self.timing.append((t0, t1))
        m.trim_many(req_ids)
        return InFlight(batch, bk, turn, B, raw)

    def collect(self, flight: "InFlight"):
        """Waits for a launched step's results: (tokens, raw log-probs, processed log-probs, logits or None)."""
        bk, B = flight.bucket, flight.n
        bk.out_done[flight.turn].synchronize()
        lp = bk.lp_host[flight.turn]
        return bk.tok_host[flight.turn][:B].tolist(), lp[0, :B].tolist(), lp[1, :B].tolist(), flight.raw


class InFlight:
    """A decode step that has been launched and whose results have not been read yet."""

    def __init__(self, batch: list[Scheduled], bucket: _Bucket, turn: int, n: int, raw) -> None:
        self.batch, self.bucket, self.turn, self.n, self.raw = batch, bucket, turn, n, raw
        self.sampling = batch            # every row samples
        self.tok_dev = bucket.out_token  # where the sampled tokens lie until the bucket's next replay

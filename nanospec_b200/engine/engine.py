"""The Python entry point: `Engine(model, EngineConfig(...)).generate(prompts, params)`.

Same surface as the reference's `Engine` (engine/engine.py:51,141-153,195): `add` a prompt of
token ids with `SamplingParams`, `step` until `sched.has_work` is false, or `generate` for
both; token ids in and out, no tokenizer inside.  One step = one call of the step function
on whatever the scheduler composed (decode tokens beside portions of prompts), then the
head projection and sampling over the rows that end a request's known tokens, in chunks of
`head_chunk` rows, with one device-to-host read per step (engine/engine.py:370-406 there).
"""

from __future__ import annotations

import time

import numpy as np
import torch

from .. import ops
from ..config.engine import EngineConfig
from ..parts.model import DecoderModel
from .scheduler import Request, SamplingParams, Scheduled, Scheduler, TokenInfo
from .graphs import InFlight
from .step import ModelRunner, StepEntry


class Engine:
    def __init__(self, model: DecoderModel, config: EngineConfig) -> None:
        self.model = model
        self.config = config
        self.device, self.dtype = model.device, model.dtype
        max_requests = config.max_running or min(config.num_blocks, 1024)
        self.runner = ModelRunner(model, config.num_blocks, config.block_size, max_requests)
        self.cache = self.runner.manager
        self.sched = Scheduler(self.cache, config.max_admit, config.max_running, config.max_step_tokens,
                               config.prefill_chunk, config.admission)
        self.eos = set(model.recipe.eos_token_ids)
        self._next_id = 0
        self.prof: dict[str, list[float]] = {}
        self._events: list[tuple[str, torch.cuda.Event]] = []
        self.steps = 0
        self.graphs = None
        if config.cuda_graphs:
            from .graphs import DecodeGraphs

            self.graphs = DecodeGraphs(self.runner, config.graph_buckets, config.record_logits)
            if config.capture_at_start:
                self.graphs.capture_all(max_requests)
        self._inflight = None  # a step that has been launched and not yet read
        self._score_bufs: list = [None, None]
        self._score_turn = 0
        self.launched_ahead = 0  # steps that were launched before their predecessor had been read
        # set to a list to have every launched step noted as (tokens, cache positions its requests hold after it,
        # rows sampled, query-key pairs under the causal mask): what a measurement needs to set a workload's time
        # against its flops and bytes
        self.step_log: list[tuple[int, int, int, int]] | None = None
        self.d2h_bytes_last = 0
        # host seconds spent composing batches (scheduler) and launching them (step description, copies, kernel
        # launches), summed over the steps; neither includes waiting for the GPU
        self.host_compose_s = 0.0
        self.host_launch_s = 0.0

    # ---- profiling (CUDA events per phase, read once per step) -------------------------------
    def _mark(self, name: str) -> None:
        if self.config.profile:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._events.append((name, e))

    def _flush_prof(self) -> None:
        if not self._events:
            return
        torch.cuda.synchronize()
        for (_, ea), (b, eb) in zip(self._events, self._events[1:]):
            self.prof.setdefault(b, []).append(ea.elapsed_time(eb))
        self._events.clear()

    # ---- requests ---------------------------------------------------------------------------
    def add(self, prompt_ids: list[int], params: SamplingParams = SamplingParams()) -> Request:
        vocab = self.model.vocab_size
        for t in prompt_ids:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        if len(prompt_ids) + params.max_tokens - 1 > self.runner.max_positions:
            raise ValueError(f"prompt of {len(prompt_ids)} tokens plus {params.max_tokens} new ones exceeds the "
                             f"model's {self.runner.max_positions} positions")
        req = Request(self._next_id, list(prompt_ids), params)
        self._next_id += 1
        self.sched.add(req)
        return req

    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams] = SamplingParams()) -> list[list[int]]:
        plist = params if isinstance(params, list) else [params] * len(prompts)
        reqs = [self.add(p, sp) for p, sp in zip(prompts, plist)]
        while self.sched.has_work:
            self.step()
        ops.check_kernel_errors(self.device)
        return [r.out_tokens for r in reqs]

    def update_weights(self, state: dict[str, torch.Tensor]) -> None:
        """Copies new weights in place (checkpoint names; see `weights.update_weights`) and restarts every running
        request from its prompt plus what it has emitted: its cache was computed by the old weights.  The reference's
        `Engine.update_weights` (engine/engine.py:167-176 there).  A step that was launched ahead is dropped."""
        from ..weights import update_weights

        update_weights(self.model, state)
        for req in list(self.sched.running):
            self.sched.restart(req)
        self._inflight = None

    def _emit(self, req: Request, info: TokenInfo) -> bool:
        """Appends the token; True when the request is done (the end token is kept in the output)."""
        req.out_tokens.append(info.token)
        if req.params.logprobs:
            req.logprobs.append(info)
        stop = info.token in self.eos and not req.params.ignore_eos
        return stop or len(req.out_tokens) >= req.params.max_tokens

    # ---- one step ---------------------------------------------------------------------------
    def step(self) -> list[Request]:
        """Composes a batch, runs it, samples; returns the requests that finished.

        Decode-only batches of up to the largest bucket go through CUDA graphs.  While nobody can be
        admitted, the step after this one is composed and launched before this one's tokens have
        reached the host: it takes them on the device, and the host's work (composing the batch,
        launching its kernels) overlaps the GPU.  A request that turns out to have ended meanwhile
        simply ignores the extra step's result."""
        if self._inflight is not None and not any(s.req.state == "running" for s in self._inflight.batch):
            self._inflight = None  # a step launched ahead for requests that have all ended meanwhile: nothing to read
        t0 = time.perf_counter()
        if self._inflight is None:
            batch = self.sched.next_batch()
            if not batch:
                return []
            self._mark("start")
            t1 = time.perf_counter()
            self._inflight = self._launch(batch, None)
            self.host_compose_s += t1 - t0
            self.host_launch_s += time.perf_counter() - t1
        flight = self._inflight
        ahead = None
        t0 = time.perf_counter()
        nxt = self._batch_ahead(flight)
        if nxt is not None:
            t1 = time.perf_counter()
            ahead = self._launch(nxt, flight)
            self.launched_ahead += 1
            self.host_compose_s += t1 - t0
            self.host_launch_s += time.perf_counter() - t1
        finished = self._collect(flight)
        self._inflight = ahead
        self._after_step()
        return finished

    def _launch(self, batch: list[Scheduled], prev):
        """Launches the step and returns a handle to collect it with.  `prev`: the step in flight whose
        sampled tokens this one takes on the device (entries with `from_row`), or None."""
        # Rows in the order in which the decode attention kernel's blocks are scheduled: the requests with the most keys
        # first, so that no long one starts when the others are done (continuous batching at the 3B shape, contexts of
        # 16 to 2,300 tokens: 13,850 against 13,250 output tokens / s).  Portions of prompts keep their order behind them.
        batch = sorted(batch, key=lambda s: -s.req.committed if len(s.tokens) == 1 else 1)
        if self.step_log is not None:
            self.step_log.append((sum(len(s.tokens) for s in batch), sum(s.req.committed + len(s.tokens) for s in batch),
                                  sum(1 for s in batch if s.samples),
                                  sum(len(s.tokens) * (2 * s.req.committed + len(s.tokens) + 1) // 2 for s in batch)))
        if self.graphs is not None and self.graphs.can_run(batch):
            take = None if prev is None else (prev.tok_dev, [s.from_row for s in batch])
            flight = self.graphs.launch(batch, self._uniforms(batch), take)
            for s in batch:
                s.req.committed += 1
            return flight
        sampling = [s for s in batch if s.samples]
        entries = [StepEntry(s.req.id, s.tokens, [len(s.tokens) - 1] if s.samples else []) for s in batch]
        take = None
        if prev is not None:
            dst, src, row = [], [], 0
            for s in batch:
                if s.from_row is not None:
                    dst.append(row)
                    src.append(s.from_row)
                row += len(s.tokens)
            take = (dst, prev.tok_dev, src)
        # the sampling options of the rows that sample travel with the step's description: [temperature | top_k |
        # top_p | uniform], one value per row each (floats by their bits)
        R = len(sampling)
        options = np.empty(4 * R, dtype=np.int32)
        as_f32 = options.view(np.float32)
        as_f32[:R] = [s.req.params.temperature for s in sampling]
        options[R: 2 * R] = [s.req.params.top_k for s in sampling]
        as_f32[2 * R: 3 * R] = [s.req.params.top_p for s in sampling]
        as_f32[3 * R:] = self._uniforms(sampling)
        ctx, want_rows, _ = self.runner.build_context(entries, take, options)
        hidden = self.runner.forward(ctx, want_rows)
        self._mark("forward")
        for s in batch:
            s.req.committed += len(s.tokens)
        return self._score_launch(hidden, batch, sampling, ctx.extras["extra"])

    def _collect(self, flight) -> list[Request]:
        """Waits for the step's tokens and hands them to their requests."""
        if isinstance(flight, InFlight):
            tok, lpr, lpp, raw = self.graphs.collect(flight)
            sampling = flight.batch
        else:
            tok, lpr, lpp, raw = self._score_collect(flight)
            sampling = flight.sampling
        self._mark("score")
        finished = []
        for row, s in enumerate(sampling):
            req = s.req
            if req.state != "running":
                continue  # it ended in the step before; this step ran for it in vain
            if raw is not None:
                req.step_logits.append(raw[row])
            if self._emit(req, TokenInfo(tok[row], lpr[row], lpp[row])):
                self.sched.finish(req)
                finished.append(req)
        return finished

    def _batch_ahead(self, flight) -> list[Scheduled] | None:
        """The batch that follows the step in flight if every request that it samples for goes on, or
        None when that cannot be said without its tokens (then the next step is composed by the
        scheduler, after this one has been collected)."""
        cfg = self.config
        if not cfg.lookahead or cfg.record_logits or cfg.profile:
            return None
        if self.sched.could_admit():
            # Somebody waits who fits: the scheduler composes the next batch, admissions included, on the assumption
            # that every request of the step in flight goes on.  (With optimistic admission it declines: composing
            # could take pages back from a request whose tokens are not known yet.)
            running = self.sched.running
            if len(flight.batch) != len(running) or any(s.req.state != "running" for s in flight.batch):
                return None
            rows = {id(s): i for i, s in enumerate(flight.sampling)}
            return self.sched.next_batch(ahead={id(s.req): rows[id(s)] for s in flight.batch if s.samples}) or None
        cache, running = self.cache, self.sched.running
        # every running request is in the step in flight; the next batch has them in the scheduler's order
        # (decoding ones first, then portions, each oldest first), and everything must fit
        if len(flight.batch) != len(running) or any(s.req.state != "running" for s in flight.batch):
            return None
        row_of = {id(s): i for i, s in enumerate(flight.sampling)}
        age = {id(r): i for i, r in enumerate(running)}
        decoding, portions = [], []
        for s in flight.batch:
            req = s.req
            if id(req) not in age:
                return None
            if not s.samples:
                portions.append(req)
            elif len(req.out_tokens) + 1 < req.params.max_tokens:  # else it ends with the step in flight
                if req.committed + 1 > self.runner.max_positions:
                    return None
                decoding.append(Scheduled(req, [0], True, from_row=row_of[id(s)]))
        decoding.sort(key=lambda sch: age[id(sch.req)])
        portions.sort(key=lambda r: age[id(r)])
        budget = cfg.max_step_tokens
        free, planned = cache.free_pages(), [0] * len(cache.groups)

        def fits(req: Request, n: int) -> bool:
            need = cache.need_between(req.committed, req.committed + n)
            if any(nd + pl > fr for nd, pl, fr in zip(need, planned, free)):
                return False
            for i, nd in enumerate(need):
                planned[i] += nd
            return True

        out: list[Scheduled] = []
        for sch in decoding:
            if budget <= 0 or not fits(sch.req, 1):
                return None
            out.append(sch)
            budget -= 1
        for req in portions:
            n = min(req.pending, cfg.prefill_chunk, budget)
            if n <= 0 or not fits(req, n):
                return None
            out.append(Scheduled(req, req.token_slice(req.committed, req.committed + n), samples=(n == req.pending)))
            budget -= n
        return out or None

    def _after_step(self) -> None:
        self.steps += 1
        if self.steps % 64 == 0:
            ops.check_kernel_errors(self.device)  # a timed-out wait inside a kernel must not pass silently
        self._flush_prof()

    def _uniforms(self, sampling: list[Scheduled]) -> list[float]:
        # one uniform per sampled token from the request's own generator (engine/engine.py:283 in
        # the reference): results do not depend on what else is in the batch
        return [s.req.next_uniform() if s.req.params.temperature > 0 else 0.0 for s in sampling]

    def _score_buffers(self, rows: int):
        """Device and pinned host buffers for a step's sampled tokens and log-probs; two sets used in turn
        (a step launched ahead writes its own while the one before it is still to be read)."""
        self._score_turn ^= 1
        bufs = self._score_bufs[self._score_turn]
        if bufs is None or bufs[0].numel() < rows:
            cap = max(256, 2 * rows)
            dev = self.device
            bufs = (torch.zeros(cap, dtype=torch.int32, device=dev), torch.zeros(2, cap, dtype=torch.float32, device=dev),
                    torch.zeros(cap, dtype=torch.int32).pin_memory(), torch.zeros(2, cap, dtype=torch.float32).pin_memory(),
                    torch.cuda.Event())
            self._score_bufs[self._score_turn] = bufs
        return bufs

    def _score_launch(self, hidden: torch.Tensor | None, batch: list[Scheduled], sampling: list[Scheduled],
                      options: torch.Tensor) -> "EagerFlight":
        """Head projection and token choice for the rows of `hidden`, `head_chunk` rows at a time; the
        results start their way to the host and are read by `_score_collect`.  `options`: the rows' sampling
        options on the device, as `_launch` laid them out."""
        if hidden is None or not sampling:
            return EagerFlight(batch, [], None, None, None, None, None)
        R = hidden.shape[0]
        temp, top_k = options[:R].view(torch.float32), options[R: 2 * R]
        top_p, u = options[2 * R: 3 * R].view(torch.float32), options[3 * R: 4 * R].view(torch.float32)
        tok_dev, lp_dev, tok_host, lp_host, done = self._score_buffers(R)
        raw = [] if self.config.record_logits else None
        chunk = self.config.head_chunk
        logits_buf = self.runner.workspace.get("logits", min(chunk, R), self.model.vocab_size, torch.float32)
        for s in range(0, R, chunk):
            e = min(s + chunk, R)
            z = self.model.logits(hidden[s:e], logits_buf[: e - s])
            if raw is not None:
                raw.append(z.cpu())
            ops.sample_rows(z, temp[s:e], top_k[s:e], top_p[s:e], u[s:e], out=(tok_dev[s:e], lp_dev[0, s:e], lp_dev[1, s:e]))
        # the step's device-to-host read: tokens and two log-probs per row (each copy contiguous: a strided copy
        # between device and host goes through a temporary and blocks the host)
        tok_host[:R].copy_(tok_dev[:R], non_blocking=True)
        lp_host[0, :R].copy_(lp_dev[0, :R], non_blocking=True)
        lp_host[1, :R].copy_(lp_dev[1, :R], non_blocking=True)
        done.record()
        self.d2h_bytes_last = R * 12
        return EagerFlight(batch, sampling, tok_dev, tok_host, lp_host, done, torch.cat(raw) if raw else None)

    def _score_collect(self, flight: "EagerFlight"):
        if not flight.sampling:
            return [], [], [], None
        R = len(flight.sampling)
        flight.done.synchronize()
        return flight.tok_host[:R].tolist(), flight.lp_host[0, :R].tolist(), flight.lp_host[1, :R].tolist(), flight.raw


class EagerFlight:
    """A step of portions and decode tokens that has been launched and whose results have not been read yet."""

    def __init__(self, batch, sampling, tok_dev, tok_host, lp_host, done, raw) -> None:
        self.batch, self.sampling = batch, sampling
        self.tok_dev, self.tok_host, self.lp_host, self.done, self.raw = tok_dev, tok_host, lp_host, done, raw

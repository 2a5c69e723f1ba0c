"""The Python entry point: `Engine(model, EngineConfig(...)).generate(prompts, params)`.

Same surface as the reference's `Engine` (engine/engine.py:51,141-153,195): `add` a prompt of
token ids with `SamplingParams`, `step` until `sched.has_work` is false, or `generate` for
both; token ids in and out, no tokenizer inside.  One step = one call of the step function
on whatever the scheduler composed (decode tokens beside portions of prompts), then the
head projection and sampling over the rows that end a request's known tokens, in chunks of
`head_chunk` rows, with one device-to-host read per step (engine/engine.py:370-406 there).
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.engine import EngineConfig
from ..parts.model import DecoderModel
from .scheduler import Request, SamplingParams, Scheduled, Scheduler, TokenInfo
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
        self._inflight = None  # a decode step that has been launched and not yet read
        self.d2h_bytes_last = 0

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

        Decode-only batches go through CUDA graphs.  While nothing else is waiting, the step after
        such a batch is launched before this one's tokens have reached the host: it takes them on
        the device, and the host's work (and the graph's launch latency) overlaps the GPU.  A request
        that turns out to have ended meanwhile simply ignores the extra step's result."""
        if self._inflight is None:
            batch = self.sched.next_batch()
            if not batch:
                return []
            self._mark("start")
            if self.graphs is None or not self.graphs.can_run(batch):
                return self._run_eager(batch)
            self._inflight = self._launch_decode(batch, ids_from_device=False)
        flight = self._inflight
        ahead = None
        if self._can_look_ahead(flight.batch):
            ahead = self._launch_decode([Scheduled(s.req, [0], True) for s in flight.batch], ids_from_device=True)
        tok, lpr, lpp, raw = self.graphs.collect(flight)
        self._mark("score")
        finished = []
        for row, s in enumerate(flight.batch):
            req = s.req
            if req.state != "running":
                continue  # it ended in the step before; this step ran for it in vain
            if raw is not None:
                req.step_logits.append(raw[row])
            if self._emit(req, TokenInfo(tok[row], lpr[row], lpp[row])):
                self.sched.finish(req)
                finished.append(req)
        self._inflight = ahead
        self._after_step()
        return finished

    def _launch_decode(self, batch: list[Scheduled], ids_from_device: bool):
        flight = self.graphs.launch(batch, self._uniforms(batch), ids_from_device)
        for s in batch:
            s.req.committed += 1
        return flight

    def _can_look_ahead(self, batch: list[Scheduled]) -> bool:
        if not self.config.lookahead or self.config.record_logits or self.sched.waiting:
            return False
        for s in batch:
            req = s.req
            # still running after the step in flight, and room for one more position
            if req.state != "running" or len(req.out_tokens) + 2 > req.params.max_tokens \
                    or req.committed + 1 > self.runner.max_positions or not self.cache.can_extend(req.id, 1):
                return False
        return True

    def _run_eager(self, batch: list[Scheduled]) -> list[Request]:
        sampling = [s for s in batch if s.samples]
        entries = [StepEntry(s.req.id, s.tokens, [len(s.tokens) - 1] if s.samples else []) for s in batch]
        hidden = self.runner.run(entries)
        self._mark("forward")
        tok, lpr, lpp, raw = self._score(hidden, sampling)
        self._mark("score")
        finished = []
        row = 0
        for s in batch:
            req = s.req
            req.committed += len(s.tokens)
            if not s.samples:
                continue
            if raw is not None:
                req.step_logits.append(raw[row])
            done = self._emit(req, TokenInfo(tok[row], lpr[row], lpp[row]))
            row += 1
            if done:
                self.sched.finish(req)
                finished.append(req)
        self._after_step()
        return finished

    def _after_step(self) -> None:
        self.steps += 1
        if self.steps % 64 == 0:
            ops.check_kernel_errors(self.device)  # a timed-out wait inside a kernel must not pass silently
        self._flush_prof()

    def _uniforms(self, sampling: list[Scheduled]) -> list[float]:
        # one uniform per sampled token from the request's own generator (engine/engine.py:283 in
        # the reference): results do not depend on what else is in the batch
        return [float(torch.rand(1, generator=s.req.gen)) if s.req.params.temperature > 0 else 0.0 for s in sampling]

    def _score(self, hidden: torch.Tensor | None, sampling: list[Scheduled]):
        """Head projection and token choice for the rows of `hidden`, `head_chunk` rows at a time."""
        if hidden is None or not sampling:
            return [], [], [], None
        R = hidden.shape[0]
        dev = self.device
        P = [s.req.params for s in sampling]
        temp = torch.tensor([p.temperature for p in P], dtype=torch.float32).to(dev, non_blocking=True)
        top_k = torch.tensor([p.top_k for p in P], dtype=torch.int32).to(dev, non_blocking=True)
        top_p = torch.tensor([p.top_p for p in P], dtype=torch.float32).to(dev, non_blocking=True)
        u = torch.tensor(self._uniforms(sampling), dtype=torch.float32).to(dev, non_blocking=True)
        out = torch.empty((3, R), dtype=torch.float32, device=dev)
        raw = [] if self.config.record_logits else None
        chunk = self.config.head_chunk
        logits_buf = self.runner.workspace.get("logits", min(chunk, R), self.model.vocab_size, torch.float32)
        for s in range(0, R, chunk):
            e = min(s + chunk, R)
            z = self.model.logits(hidden[s:e], logits_buf[: e - s])
            if raw is not None:
                raw.append(z.cpu())
            tok, lpr, lpp = ops.sample_rows(z, temp[s:e], top_k[s:e], top_p[s:e], u[s:e])
            out[0, s:e] = tok
            out[1, s:e] = lpr
            out[2, s:e] = lpp
        vals = out.cpu()  # the step's one device-to-host read
        self.d2h_bytes_last = vals.numel() * 4
        tok = [int(x) for x in vals[0].tolist()]
        return tok, vals[1].tolist(), vals[2].tolist(), (torch.cat(raw) if raw else None)

"""Requests and the scheduler above the step function.  No tensors besides the per-request
random generator.

Kept from the reference (sched/scheduler.py:17-134): `SamplingParams` and `Request` with its
states, FIFO admission with head-of-line blocking, at most `max_admit` admissions per step
and `max_running` live requests, worst-case page reservation so that a running request can
always grow (`admission="reserve"`), `finish`, and `restart` (back to the head of the queue,
its cache dropped, emitted tokens kept).

Added: prompts are cut into portions under a token budget (`max_step_tokens` per step,
`prefill_chunk` per request and step), decoding requests and portions of prompts share one
step, and an optimistic admission mode in which pages can run out.  What happens then is
decided here: the newest running request is preempted - its pages and state slot are given
back, it returns to the head of the queue and is recomputed from its prompt plus the tokens
it has already emitted - until the older requests fit.  A request that could never fit in
the pool alone is refused when it is added.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import torch

from ..cache import CacheManager


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = 128     # most new tokens of the request
    temperature: float = 0.0  # zero picks the largest raw logit; otherwise logits are divided by it before the draw
    top_k: int = 0            # keep only the k most likely tokens; zero keeps all
    top_p: float = 1.0        # keep the smallest set of most likely tokens whose probability reaches this
    seed: int | None = None   # seeds the request's own generator; without one the stream is unpredictable
    logprobs: bool = False    # record a TokenInfo for every emitted token
    ignore_eos: bool = False  # keep generating past an end-of-sequence token (benchmarks on random weights)

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.temperature < 0 or self.top_k < 0 or not 0.0 <= self.top_p <= 1.0:
            raise ValueError("temperature and top_k must not be negative, top_p must lie in [0, 1]")


@dataclass(slots=True)
class TokenInfo:
    token: int
    logprob: float         # the token's log-probability under the unprocessed logits
    sample_logprob: float  # its log-probability under the distribution that the draw used (after temperature, top-k
                           # and top-p); a greedy pick records 0


@dataclass
class Request:
    id: int
    prompt_ids: list[int]
    params: SamplingParams
    out_tokens: list[int] = field(default_factory=list)
    state: str = "waiting"  # "waiting" in the queue, "running" with cache pages, "done"
    committed: int = 0      # positions of this request that the cache holds; tokens()[committed:] have not run yet
    preemptions: int = 0
    gen: torch.Generator = None  # the request's own host generator, so that what it draws is the same in any batch
    logprobs: list[TokenInfo] = field(default_factory=list)
    step_logits: list = field(default_factory=list)  # only with EngineConfig.record_logits
    peak_pages: list[int] | None = None  # the scheduler's note: most pages per cache group it can ever hold
    _uniforms: list[float] = field(default_factory=list, repr=False)  # drawn ahead from `gen`, not yet used

    def __post_init__(self) -> None:
        self.gen = torch.Generator()
        if self.params.seed is not None:
            self.gen.manual_seed(self.params.seed)
        else:
            self.gen.seed()

    def next_uniform(self) -> float:
        """The next number of the request's own stream, the one that `torch.rand(1, generator=gen)` would give
        (sched/scheduler.py:64,74-76 and engine/engine.py:283 in the reference): eight are drawn at a time, which
        gives the same stream as single draws and costs an eighth of the calls."""
        if not self._uniforms:
            self._uniforms = torch.rand(8, generator=self.gen).tolist()[::-1]
        return self._uniforms.pop()

    def tokens(self) -> list[int]:
        return self.prompt_ids + self.out_tokens

    def token_slice(self, start: int, end: int) -> list[int]:
        """tokens()[start:end] without building the whole list."""
        n_prompt = len(self.prompt_ids)
        if end <= n_prompt:
            return self.prompt_ids[start:end]
        if start >= n_prompt:
            return self.out_tokens[start - n_prompt: end - n_prompt]
        return self.prompt_ids[start:] + self.out_tokens[: end - n_prompt]

    @property
    def seq_len(self) -> int:
        return len(self.prompt_ids) + len(self.out_tokens)

    @property
    def pending(self) -> int:
        """Tokens not yet run through the model (1 while decoding)."""
        return self.seq_len - self.committed

    @property
    def final_len(self) -> int:
        """Most cache positions this request can ever hold."""
        return len(self.prompt_ids) + self.params.max_tokens - 1


@dataclass
class Scheduled:
    """One request's share of the next step."""

    req: Request
    tokens: list[int]
    samples: bool  # the portion ends at the request's last known token: its last logits give the next token
    from_row: int | None = None  # the one token is still on the device: row of the step before among its sampled rows


class RequestTooLarge(ValueError):
    pass


class Scheduler:
    def __init__(self, cache: CacheManager, max_admit: int = 32, max_running: int | None = None,
                 max_step_tokens: int = 8192, prefill_chunk: int = 2048, admission: str = "reserve") -> None:
        self.cache = cache
        self.max_admit, self.max_running = max_admit, max_running
        self.max_step_tokens, self.prefill_chunk = max_step_tokens, prefill_chunk
        self.admission = admission
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.preempted_total = 0

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- page arithmetic ------------------------------------------------------------------
    def _longest_portion(self) -> int:
        return min(self.prefill_chunk, self.max_step_tokens)

    def _peak(self, req: Request) -> list[int]:
        # a request's final length and the longest portion do not change while it lives
        if req.peak_pages is None:
            req.peak_pages = self.cache.peak_pages(req.final_len, self._longest_portion())
        return req.peak_pages

    def add(self, req: Request) -> None:
        assert req.state == "waiting"
        if not req.prompt_ids:
            raise ValueError("a request needs at least one prompt token")
        if any(p > g.pool.num_pages for p, g in zip(self._peak(req), self.cache.groups)):
            raise RequestTooLarge(
                f"request {req.id} needs up to {self._peak(req)} pages per cache group for {req.final_len} positions; "
                f"the pool has {self.cache.num_blocks}")
        self.waiting.append(req)

    # ---- one step's batch -----------------------------------------------------------------
    def next_batch(self, ahead: dict[int, int] | None = None) -> list[Scheduled] | None:
        """Decoding requests first (one token each), then portions of running prompts, then
        admissions; all under the token budget and the pages that are free.

        `ahead`: the batch is composed while a step is still in flight.  It maps id(request) to the row of that
        step that samples the request's next token: such a request brings a placeholder token that the step takes
        on the device (`Scheduled.from_row`), unless the token in flight is its last.  Requests that the step in
        flight turns out to have ended simply ignore their row of this one; admissions count them as still
        running, which errs on the safe side.  Only with worst-case reservation, where composing a batch never
        takes pages back from anybody: otherwise None is returned and nothing has changed."""
        if ahead is not None and self.admission != "reserve":
            return None
        cache = self.cache
        budget = self.max_step_tokens
        planned = [0] * len(cache.groups)  # pages this step's entries will take
        batch: list[Scheduled] = []

        free = cache.free_pages()  # what this step may take: nothing is taken or given back while it is composed
        # (a preemption gives pages back: `free` is read again after one)

        need: list[int] = []  # of the request being looked at, as `fits` last computed it

        def fits(req_id: int | None, cur: int, n: int) -> bool:
            nonlocal need
            need = cache.need_between(cur, cur + n)  # a live request holds exactly the pages of its `cur` positions
            return all(nd + pl <= fr for nd, pl, fr in zip(need, planned, free))

        def plan(req: Request, n: int) -> None:
            # follows a successful fits() for the same request and portion
            nonlocal budget
            for i, nd in enumerate(need):
                planned[i] += nd
            if ahead is not None and id(req) in ahead:
                batch.append(Scheduled(req, [0], True, from_row=ahead[id(req)]))
            else:
                toks = req.token_slice(req.committed, req.committed + n)
                batch.append(Scheduled(req, toks, samples=(n == req.pending)))
            budget -= n

        def unplan(victim: Request) -> None:
            nonlocal budget
            for k, sch in enumerate(batch):
                if sch.req is victim:
                    for gi, nd in enumerate(cache.need_between(victim.committed, victim.committed + len(sch.tokens))):
                        planned[gi] -= nd
                    budget += len(sch.tokens)
                    del batch[k]
                    return

        # 1. running requests: those that decode first (one token each), then portions of
        #    prompts, each oldest first; when pages run out the newest running request is preempted
        preempted = False

        def pending(r: Request) -> int:
            if ahead is not None and id(r) in ahead:  # its next token is being sampled: one more, unless that one is its last
                return 1 if len(r.out_tokens) + 1 < r.params.max_tokens else 0
            return r.pending

        order = [r for r in self.running if pending(r) == 1] + [r for r in self.running if pending(r) > 1]
        for req in order:
            if req.state != "running":
                continue  # preempted a moment ago
            if budget <= 0:
                break
            n = min(pending(req), self.prefill_chunk, budget)
            while not fits(req.id, req.committed, n):
                if self.admission == "reserve":
                    raise AssertionError("page reservation was violated")  # cannot happen by construction
                victim = self.running[-1]
                if victim is req:
                    if n > 1:  # the newest request itself: try a shorter portion first
                        n = max(1, n // 2)
                        continue
                    if len(self.running) == 1:
                        raise AssertionError("a single request does not fit in the pool")  # add() refuses these
                unplan(victim)
                self.preempt(victim)
                free = cache.free_pages()
                preempted = True
                if victim is req:
                    n = 0
                    break
            if n > 0:
                plan(req, n)

        # 2. admissions, FIFO with head-of-line blocking
        admitted = 0
        headroom = None
        if preempted:
            return batch  # no admission in a step that had to give pages back
        if self.admission == "reserve" and self.waiting:
            owed = [0] * len(cache.groups)
            for r in self.running:
                for gi, (pk, held) in enumerate(zip(self._peak(r), cache.held_pages(r.id))):
                    owed[gi] += max(0, pk - held)
            headroom = [f - o for f, o in zip(free, owed)]
        while (self.waiting and admitted < self.max_admit and budget > 0
               and (self.max_running is None or len(self.running) < self.max_running)
               and cache.slots.num_free > 0):
            req = self.waiting[0]
            n = min(req.pending, self.prefill_chunk, budget)
            if self.admission == "reserve":
                peak = self._peak(req)
                if any(p > h for p, h in zip(peak, headroom)):
                    break
                headroom = [h - p for h, p in zip(headroom, peak)]
                need = cache.need_between(0, n)
            elif not fits(None, 0, n):
                break
            self.waiting.popleft()
            cache.begin(req.id)
            req.state = "running"
            self.running.append(req)
            plan(req, n)
            admitted += 1
        return batch

    def could_admit(self) -> bool:
        """Whether `next_batch` would admit the head of the queue as things stand now (live requests,
        state slots, pages).  The engine asks before it launches a step ahead of its predecessor's
        results: while nobody can be admitted anyway, the next batch does not depend on them."""
        if not self.waiting:
            return False
        if self.max_running is not None and len(self.running) >= self.max_running:
            return False
        cache = self.cache
        if cache.slots.num_free <= 0:
            return False
        req = self.waiting[0]
        free = cache.free_pages()
        if self.admission == "reserve":
            owed = [0] * len(cache.groups)
            for r in self.running:
                for gi, (pk, held) in enumerate(zip(self._peak(r), cache.held_pages(r.id))):
                    owed[gi] += max(0, pk - held)
            return all(p <= f - o for p, f, o in zip(self._peak(req), free, owed))
        n = min(req.pending, self.prefill_chunk, self.max_step_tokens)
        return all(nd <= fr for nd, fr in zip(cache.need_between(0, n), free))

    # ---- transitions -----------------------------------------------------------------------
    def finish(self, req: Request) -> None:
        self.running.remove(req)
        self.cache.end(req.id)
        req.state = "done"

    def preempt(self, req: Request) -> None:
        """Pages ran out: drop the request's cache and put it back at the head of the queue.
        It is recomputed from its prompt plus the tokens it has emitted, which are kept."""
        self.restart(req)
        req.preemptions += 1
        self.preempted_total += 1

    def restart(self, req: Request) -> None:
        """Back to the head of the queue with nothing cached (the reference's `restart`,
        sched/scheduler.py:128-134, used there after a weight swap)."""
        self.running.remove(req)
        self.cache.end(req.id)
        req.state, req.committed = "waiting", 0
        self.waiting.appendleft(req)

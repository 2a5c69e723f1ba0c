"""Engine options. Names and meanings follow the reference's `EngineConfig`
(engine/engine.py:30-47) where it has them: `num_blocks`, `block_size`, `max_admit`,
`max_running`, `cuda_graphs`, `record_logits`, `profile`, `head_chunk`.  The reference
prefills a prompt whole in its admission step; `max_step_tokens`, `prefill_chunk` and
`admission` are this engine's own additions for portions of prompts under a token budget.
As there (engine/engine.py:74,97-106) the decode graphs are captured when the engine is
built, so that no request pays for a capture; `capture_at_start=False` leaves each bucket
to its first use.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class EngineConfig:
    num_blocks: int                      # pages in every cache group's pool
    block_size: int = 16                 # tokens per page
    max_admit: int = 32                  # admissions per step
    max_running: int | None = None       # live requests; None = whatever the pool holds
    cuda_graphs: bool = True             # replay decode-only steps from captured graphs
    record_logits: bool = False          # keep each request's per-step next-token logits on the host
    profile: bool = False                # per-phase CUDA-event timings in Engine.prof
    head_chunk: int = 256                # rows per head-projection + sampling chunk
    max_step_tokens: int = 8192          # token budget of one step (decode tokens count 1 each)
    prefill_chunk: int = 2048            # longest portion of one prompt in one step
    admission: str = "reserve"           # "reserve": worst-case page reservation, never preempts;
                                         # "optimistic": admit on current need, preempt the newest when pages run out
    graph_buckets: tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64, 128, 256)  # the reference stops at 64 (engine/graphs.py:22)
    lookahead: bool = True               # launch the next decode step before the last one's tokens reach the host
    capture_at_start: bool = True        # capture every bucket's graph when the engine is built, not at first use

    def __post_init__(self) -> None:
        if self.num_blocks <= 0 or self.block_size <= 0:
            raise ValueError("num_blocks and block_size must be positive")
        if self.admission not in ("reserve", "optimistic"):
            raise ValueError(f"unknown admission policy {self.admission!r}")
        if self.max_step_tokens < 1 or self.prefill_chunk < 1 or self.max_admit < 1 or self.head_chunk < 1:
            raise ValueError("max_step_tokens, prefill_chunk, max_admit and head_chunk must be at least 1")
        if self.max_running is not None and self.max_running < 1:
            raise ValueError("max_running must be at least 1 when given")

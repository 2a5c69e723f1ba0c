"""What a part sees of one step: the flattened batch, the cache lane it works on, and
scratch buffers.  Built by the engine (engine/step.py), read by the parts."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class LaneView:
    """One cache lane as a mixer sees it during a step."""

    k: torch.Tensor | None            # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor | None
    block_table: torch.Tensor | None  # [requests, max_pages] int32: page of each logical block
    page_size: int
    window: int = 0
    state: torch.Tensor | None = None  # [slots, *state_shape] when the mixer asked for state


class Workspace:
    """Scratch activations keyed by (name, columns, dtype), sized for the largest step seen.
    Buffers are reused by every layer, so a model's activations cost one layer's worth."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self._bufs: dict[tuple[str, int, torch.dtype], torch.Tensor] = {}
        self.frozen = False  # set while CUDA graphs hold pointers into the buffers

    def get(self, name: str, rows: int, cols: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """`zero`: the buffer is zero-filled when it is (re)allocated - for scratch that its
        kernel leaves zeroed after every use."""
        key = (name, cols, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[0] < rows:
            if self.frozen and buf is not None:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while CUDA graphs point into it")
            cap = max(rows, 16 if buf is None else 2 * buf.shape[0])
            make = torch.zeros if zero else torch.empty
            buf = make((cap, cols), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:rows]

    def reserve(self, rows: int) -> None:
        """Grows every buffer seen so far to hold `rows` rows."""
        for (name, cols, dtype), buf in list(self._bufs.items()):
            if buf.shape[0] < rows:
                self._bufs[(name, cols, dtype)] = torch.empty((rows, cols), dtype=dtype, device=self.device)


@dataclass
class StepContext:
    """One step's batch, flattened: N tokens of B requests.

    Device tensors are int32.  Token n belongs to request `token_req[n]` (row of the block
    tables; negative = padding row, skipped by every kernel) and sits at `positions[n]` of
    its sequence.  Request b's tokens are rows qo_indptr[b] .. qo_indptr[b+1] and after this
    step it holds kv_len[b] positions.  `state_slot[b]` is its slot of fixed-size state.

    What a mixer with state may rely on.  `lane.state` is [slots + 1, *shape]; request b's state is
    `lane.state[state_slot[b]]`, zero when the request brings its first tokens, and the mixer leaves in it
    the state after the request's last token of this step.  In a decode step replayed from a CUDA graph
    only the device tensors are current: `q_lens`, `kv_lens` and `state_slots_host` are fixed at capture
    (every request brings one token) and `state_slots_host` is empty, so a mixer that wants to run under
    graphs addresses its state through `state_slot`, `token_req` and `qo_indptr` on the device.  Padding
    rows (token_req < 0) carry the scratch slot, the last one, which no request holds: they may be read
    and written like any other and need no mask.
    """

    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_req: torch.Tensor
    qo_indptr: torch.Tensor
    kv_len: torch.Tensor
    state_slot: torch.Tensor
    q_lens: list[int]
    kv_lens: list[int]
    lanes: list[LaneView]
    workspace: Workspace
    dtype: torch.dtype
    device: torch.device
    max_q_len: int = 0
    max_kv_len: int = 0
    state_slots_host: list[int] = field(default_factory=list)  # host copy of state_slot
    extras: dict = field(default_factory=dict)

    def buffer(self, name: str, cols: int, dtype: torch.dtype | None = None, rows: int | None = None) -> torch.Tensor:
        return self.workspace.get(name, self.n_tokens if rows is None else rows, cols, dtype or self.dtype)

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1

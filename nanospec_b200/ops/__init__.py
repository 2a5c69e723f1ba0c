"""Python faces of the CUDA kernels.  Each function checks its tensors (device, dtype,
layout) and launches on the current CUDA stream; none of them has a CPU or library path
except `linear` in bfloat16, which may hand a plain matrix product to cuBLAS.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import lib
from .lib import KernelError

F32, BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dt}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)  # the handle without a Stream object around it


def _stream() -> int:
    """The current CUDA stream of the current device, as the integer that the C ABI takes (asked for
    at every launch, so that stream contexts and graph captures are followed)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must live on a CUDA device; there is no CPU path")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _i32(t: torch.Tensor | None, name: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n] = float(table[ids[n]]); out is the fp32 residual stream [N, hidden]."""
    _cuda(table, ids, out)
    _i32(ids, "ids")
    n, hidden = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed: out must be contiguous float32 and the table contiguous")
    if table.shape[1] != hidden or ids.numel() != n:
        raise KernelError(f"embed: table {tuple(table.shape)}, ids {ids.numel()}, out {tuple(out.shape)} do not agree")
    lib.call("ns_embed", table.data_ptr(), ids.data_ptr(), out.data_ptr(), n, hidden, table.shape[0],
             dtype_code(table.dtype), _stream())
    return out


def take_ids(ids: torch.Tensor, dst_rows: torch.Tensor, src: torch.Tensor, src_rows: torch.Tensor) -> None:
    """ids[dst_rows[i]] = src[src_rows[i]]: a step takes, on the device, the tokens that the step before it sampled."""
    _cuda(ids, dst_rows, src, src_rows)
    for t, name in ((ids, "ids"), (dst_rows, "dst_rows"), (src, "src"), (src_rows, "src_rows")):
        _i32(t, name)
    if dst_rows.numel() != src_rows.numel():
        raise KernelError("take_ids: one source row per destination row")
    lib.call("ns_take_ids", ids.data_ptr(), dst_rows.data_ptr(), src.data_ptr(), src_rows.data_ptr(), dst_rows.numel(), _stream())


def add_rmsnorm(resid: torch.Tensor, branch: torch.Tensor | None, gain: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None, write_resid: bool = True) -> torch.Tensor:
    """resid (+= branch); out = rmsnorm(resid) * gain.  With `rows`, output row j reads
    input row rows[j] and the residual is left unchanged."""
    _cuda(resid, branch, gain, out, rows)
    _i32(rows, "rows")
    hidden = resid.shape[1]
    n_rows = out.shape[0]
    if resid.dtype != torch.float32 or gain.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream and the gain are float32")
    if not (resid.is_contiguous() and out.is_contiguous() and gain.is_contiguous()) or out.shape[1] != hidden \
            or gain.numel() != hidden:
        raise KernelError("add_rmsnorm: operands must be contiguous and agree on the width")
    if branch is not None and (branch.dtype != out.dtype or branch.shape != resid.shape or not branch.is_contiguous()):
        raise KernelError("add_rmsnorm: the branch must match the residual's shape and the output's dtype")
    if rows is None and n_rows != resid.shape[0]:
        raise KernelError("add_rmsnorm: out and resid differ in rows")
    if rows is not None:
        if rows.numel() != n_rows:
            raise KernelError("add_rmsnorm: one row index per output row")
        write_resid = False
    lib.call("ns_add_rmsnorm", resid.data_ptr(), _ptr(branch), gain.data_ptr(), out.data_ptr(), _ptr(rows), n_rows,
             hidden, float(eps), int(bool(write_resid)), dtype_code(out.dtype), _stream())
    return out


def residual_add(resid: torch.Tensor, branch: torch.Tensor) -> torch.Tensor:
    _cuda(resid, branch)
    if resid.dtype != torch.float32 or resid.shape != branch.shape or not (resid.is_contiguous() and branch.is_contiguous()):
        raise KernelError("residual_add: float32 residual and a branch of the same shape, both contiguous")
    lib.call("ns_residual_add", resid.data_ptr(), branch.data_ptr(), resid.shape[0], resid.shape[1],
             dtype_code(branch.dtype), _stream())
    return resid


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> torch.Tensor:
    """out[n, j] = silu(gate_up[n, j]) * gate_up[n, I + j]; with `block` > 0 gate and up alternate in
    runs of `block` features instead (gate j at (j // block) * 2 * block + j % block, up `block` further)."""
    _cuda(gate_up, out)
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter) or gate_up.dtype != out.dtype or not (gate_up.is_contiguous() and out.is_contiguous()):
        raise KernelError("swiglu: gate_up must be [N, 2I] and out [N, I], same dtype, contiguous")
    lib.call("ns_swiglu", gate_up.data_ptr(), out.data_ptr(), n, inter, int(block), dtype_code(out.dtype), _stream())
    return out


class _TensorCoreGemmState:
    """Per-device state of the tcgen05 matrix product: the flag that a timed-out wait sets."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.error = torch.zeros(1, dtype=torch.int32, device=device)


_tc_state: dict[torch.device, _TensorCoreGemmState] = {}
_sm_counts: dict[int, int] = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200): the one place the launch heuristics
    below take the size of the chip from."""
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return n


USE_TENSOR_CORE_GEMM = True  # the hand-written tcgen05 kernel; False hands every bf16 product to cuBLAS
# Products with more tokens than this go to cuBLAS, whose kernels are ahead of the hand-written
# one there (measured in decode steps of the 8B shape with 1,024 tokens of context: with 32 tokens the
# hand-written kernel and its fused epilogues take 3.64 ms against 4.40 ms, with 48 tokens 4.71 ms against
# 4.80 ms, with 64 tokens 4.79 ms against 4.96 ms; at 2,048 tokens it reaches 68-85 % of cuBLAS); None = no limit.
TENSOR_CORE_GEMM_MAX_TOKENS: int | None = 64


def _tc(device: torch.device) -> _TensorCoreGemmState:
    st = _tc_state.get(device)
    if st is None:
        st = _tc_state[device] = _TensorCoreGemmState(device)
    return st


def set_programmatic_launch(enabled: bool) -> None:
    """Kernels may overlap the tail of their predecessor in the stream (default on)."""
    lib.call("ns_set_pdl", int(bool(enabled)))


def check_kernel_errors(device: torch.device | None = None) -> None:
    """Raises if a kernel recorded a timed-out wait since the last check (one small device read)."""
    for dev, st in _tc_state.items():
        if device is not None and dev != device:
            continue
        code = int(st.error.item())
        if code:
            st.error.zero_()
            what = {1: "matrix product: the TMA producer waited for a free stage", 2: "matrix product: the MMA issuer waited for a tile",
                    3: "matrix product: the epilogue waited for the accumulator", 4: "matrix product: copies in flight did not land",
                    11: "prefill attention: the loader waited for a free stage", 12: "prefill attention: the MMA issuer waited",
                    13: "prefill attention: a softmax warp waited", 21: "decode attention: the loader waited for a free stage",
                    22: "decode attention: a warp waited for its keys",
                    31: "wait probe: nobody arrives at its barrier"}.get(code, "?")
            raise KernelError(f"a kernel gave up waiting on an mbarrier (the limit is two seconds) - {what} (code {code}); "
                              "its output is not valid")


def wait_probe(device: torch.device, limit_ns: int = 1_000_000) -> bool:
    """Launches the one-block kernel of csrc/wait_probe.cu, whose only thread waits `limit_ns` on a barrier at
    which nobody arrives, gives up and records its code in the device's error word, as the production kernels'
    bounded waits do.  Returns whether the wait completed (it cannot); `check_kernel_errors` raises afterwards."""
    st = _tc(torch.device(device) if not isinstance(device, torch.device) else device)
    ok = torch.full((1,), -1, dtype=torch.int32, device=st.device)
    lib.call("ns_wait_probe", st.error.data_ptr(), int(limit_ns), ok.data_ptr(), _stream())
    return bool(ok.item() == 1)


def gemm_splits(M: int, N: int, K: int) -> int:
    """How many blocks share the k range of one output tile: enough to occupy the SMs when the
    output has few tiles (a decode step), 1 when it has many."""
    tokens_per_block = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
    tiles = -(-N // 128) * -(-M // tokens_per_block)
    k_blocks = -(-K // 64)
    resident = sm_count() * (2 if tokens_per_block <= 64 else 1)
    # a block keeps at least 8 k blocks of 64, or 4 in steps of up to 16 tokens, whose six stages then hold a block's
    # whole share of a small matrix before the step's predecessor has finished (measured at the 1B shape, 8 requests:
    # 0.865 ms per step against 0.887; at 64 requests the finer split costs 2 %)
    def splits_with(min_k_blocks: int) -> int:
        want = max(1, min(8, resident // tiles, k_blocks // min_k_blocks))
        return 1 << (want.bit_length() - 1)  # the blocks of a tile form a cluster of 1, 2, 4 or 8

    splits = splits_with(4 if M <= 16 else 8)
    if tiles * splits < sm_count():
        # fewer blocks than SMs (the 3B shape's output projection at 64 requests: 24 tiles x 4 blocks): the finer split
        # after all (continuous batching at that shape: 13,290 against 13,200 output tokens / s)
        splits = splits_with(4)
    return splits


def linear_tensor_core(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: int | None = None) -> bool:
    """The tcgen05 kernel (csrc/gemm_tcgen05.cu).  Returns False, having done nothing, when the
    operands do not meet TMA's rules (K and the row strides multiples of 8 elements, 16-byte bases)."""
    M, K = x.shape
    N = w.shape[0]
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 \
            or x.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    st = _tc(x.device)
    if splits is None:
        splits = gemm_splits(M, N, K)
    lib.call("ns_gemm_bf16_tc", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0),
             out.stride(0), int(out.dtype == torch.float32), splits, st.error.data_ptr(), _stream())
    return True


FUSE_NORM = True  # a decode step's products take over the residual sum and the norm that follows them


@dataclass
class NormSink:
    """Where a product's output goes when the residual sum and the RMSNorm that follow are folded
    into its epilogue: `resid` [N, H] float32 is updated in place, `gain` [H] and `eps` are the norm's."""

    resid: torch.Tensor
    gain: torch.Tensor
    eps: float
    workspace: object  # parts.context.Workspace: the buffers of the result come from it


@dataclass
class RowScaled:
    """Normed activations that still lack the norm's scale: `x` [N, H] = gain * resid in the compute
    dtype and `partials` [N, P] float32, per-row partial sums of resid^2.  Row n's scale is
    rsqrt(sum(partials[n]) / hidden + eps); the product that reads `x` applies it to its output rows
    (a product is linear in a per-row scale of its input).  `gain` identifies the norm it stands for."""

    x: torch.Tensor
    partials: torch.Tensor
    hidden: int
    eps: float
    gain: torch.Tensor

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype


def _tma_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    K = x.shape[1]
    return not (K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.stride(1) != 1 or w.stride(1) != 1
                or x.data_ptr() % 16 or w.data_ptr() % 16)


def norm_fusion_ok(n_tokens: int, dtype: torch.dtype, *weights: torch.Tensor) -> bool:
    """Whether a step of `n_tokens` in `dtype` may hand normed activations on as `RowScaled` to products
    with these weights (and fold a norm into a product with them): the tcgen05 kernel with a tile of up to 64
    tokens, feature counts in multiples of 128, rows that TMA can address."""
    if not (FUSE_NORM and USE_TENSOR_CORE_GEMM and dtype == torch.bfloat16 and 0 < n_tokens <= 64):
        return False
    if TENSOR_CORE_GEMM_MAX_TOKENS is not None and n_tokens > TENSOR_CORE_GEMM_MAX_TOKENS:
        return False
    return all(w.dtype == torch.bfloat16 and w.shape[0] % 128 == 0 and w.shape[1] % 8 == 0 and w.stride(1) == 1
               and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0 for w in weights)


def _linear_norm(x, w: torch.Tensor, out: torch.Tensor | None, gated: bool, sink: NormSink | None):
    """The tcgen05 product with the norm epilogues: x a tensor or RowScaled; returns `out`, or the
    RowScaled that the sink produced."""
    scaled = x if isinstance(x, RowScaled) else None
    xt = scaled.x if scaled is not None else x
    M, K = xt.shape
    N = w.shape[0]
    if w.shape[1] != K or not _tma_ok(xt, w) or M > 64:
        raise KernelError(f"linear: the norm epilogues cannot take x {tuple(xt.shape)}, w {tuple(w.shape)}")
    splits = gemm_splits(M, N, K)
    res = None
    if sink is not None:
        if gated or N % 128 or sink.resid.shape != (M, N) or not sink.resid.is_contiguous():
            raise KernelError("linear: a norm sink takes an ungated product whose width is the residual's, a multiple of 128")
        ws = sink.workspace
        res = RowScaled(ws.get("sink_x", M, N, torch.bfloat16), ws.get("sink_partials", M, (N // 128) * splits, torch.float32),
                        N, sink.eps, sink.gain)
    elif out is None or out.shape != (M, N // 2 if gated else N) or out.stride(1) != 1:
        raise KernelError("linear: the output does not fit the product")
    lib.call("ns_gemm_bf16_tc_norm", xt.data_ptr(), w.data_ptr(), _ptr(out), M, N, K, xt.stride(0), w.stride(0),
             out.stride(0) if out is not None else 0, int(out is not None and out.dtype == torch.float32), splits, int(gated),
             _ptr(scaled.partials if scaled is not None else None), scaled.partials.shape[1] if scaled is not None else 0,
             scaled.hidden if scaled is not None else 0, float(scaled.eps) if scaled is not None else 0.0,
             _ptr(sink.resid if sink is not None else None), _ptr(sink.gain if sink is not None else None),
             _ptr(res.x if res is not None else None), _ptr(res.partials if res is not None else None),
             N if sink is not None else 0, _tc(xt.device).error.data_ptr(), _stream())
    return res if res is not None else out


def linear(x, w: torch.Tensor, out: torch.Tensor, sink: NormSink | None = None):
    """out[M, N] = x[M, K] @ w[N, K]^T with fp32 accumulation.

    `x` may be a `RowScaled` (its rows' scale is applied to the output).  With a `sink` that the product
    can fold in (`norm_fusion_ok`), nothing is written to `out`: the residual is updated and a `RowScaled`
    for the norm that follows is returned; otherwise `out` is returned and the caller runs the norm.

    float32: the CUDA-core kernel (true fp32, k-ascending sums, independent of M).
    bfloat16: the tcgen05 kernel; operands that TMA cannot address (K or a row stride that is no
    multiple of 8) are a plain matrix product for cuBLAS, as the reference hands its `nn.Linear`
    calls to it (model/llama.py:175,184,195).  `out` may be bfloat16 or float32.
    """
    if isinstance(x, RowScaled) or (sink is not None and norm_fusion_ok(x.shape[0], x.dtype, w)
                                    and sink.resid.shape[1] == w.shape[0] and _tma_ok(x, w)):
        return _linear_norm(x, w, out, False, sink)
    _cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype == torch.float32:
        if w.dtype != torch.float32 or out.dtype != torch.float32:
            raise KernelError("linear: a float32 product takes float32 weights and output")
        if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear: operands must be row-major")
        lib.call("ns_gemm_f32", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0),
                 out.stride(0), _stream())
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported operand types {x.dtype}, {w.dtype}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"linear: unsupported output type {out.dtype}")
    if USE_TENSOR_CORE_GEMM and (TENSOR_CORE_GEMM_MAX_TOKENS is None or M <= TENSOR_CORE_GEMM_MAX_TOKENS) \
            and linear_tensor_core(x, w, out):
        return out
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    return out


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int, nq: int,
                  nkv: int, head_dim: int, write_kv: bool = True) -> None:
    """Rotates q and k of the packed [q | k | v] rows in place / into the cache, stores v."""
    _cuda(qkv, positions, token_req, block_table, inv_freq, k_cache, v_cache)
    _i32(positions, "positions"), _i32(token_req, "token_req")
    n = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * head_dim or not qkv.is_contiguous():
        raise KernelError("rope_kv_write: qkv must be contiguous [N, (nq + 2 nkv) * head_dim]")
    if block_table.dtype != torch.int32 or block_table.stride(1) != 1:
        raise KernelError("rope_kv_write: block_table must be int32 with unit inner stride")
    if inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous():
        raise KernelError("rope_kv_write: inv_freq must be contiguous float32")
    if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("rope_kv_write: cache pages must be contiguous and of the activations' dtype")
    lib.call("ns_rope_kv_write", qkv.data_ptr(), positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), inv_freq.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_size, nq, nkv,
             head_dim, inv_freq.numel(), n, int(bool(write_kv)), dtype_code(qkv.dtype), _stream())


FUSE_ROPE = True  # short steps rotate q and k and write k and v to the cache in the projection's epilogue


def linear_rope(x, w: torch.Tensor, out: torch.Tensor, positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                inv_freq: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int, nq: int, nkv: int,
                head_dim: int, write_kv: bool = True) -> bool:
    """The packed [q | k | v] projection with the rotation and the cache write in its epilogue
    (csrc/gemm_tcgen05.cu): out[:, : nq * head_dim] receives the rotated q; k (rotated) and v go to the cache.
    `x` may be a `RowScaled`.  Returns False, having done nothing, when the step or the sizes do not fit
    (more than 64 tokens, a head size other than 32, 64 or 128, features that do not fill tiles of 128, ...)."""
    xt = x.x if isinstance(x, RowScaled) else x
    M, K = xt.shape
    N = w.shape[0]
    if not (FUSE_ROPE and USE_TENSOR_CORE_GEMM and xt.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and 0 < M <= 64
            and (TENSOR_CORE_GEMM_MAX_TOKENS is None or M <= TENSOR_CORE_GEMM_MAX_TOKENS)
            and head_dim in (32, 64, 128) and N == (nq + 2 * nkv) * head_dim and N % 128 == 0 and w.shape[1] == K
            and _tma_ok(xt, w) and out.shape == (M, N) and out.stride(1) == 1 and k_cache.dtype == torch.bfloat16
            and k_cache.is_contiguous() and v_cache.is_contiguous() and block_table.dtype == torch.int32
            and block_table.stride(1) == 1 and inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()):
        return False
    _cuda(xt, w, out, positions, token_req, block_table, inv_freq, k_cache, v_cache)
    _i32(positions, "positions"), _i32(token_req, "token_req")
    scaled = x if isinstance(x, RowScaled) else None
    lib.call("ns_gemm_bf16_tc_rope", xt.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, xt.stride(0), w.stride(0),
             out.stride(0), gemm_splits(M, N, K), _ptr(scaled.partials if scaled is not None else None),
             scaled.partials.shape[1] if scaled is not None else 0, scaled.hidden if scaled is not None else 0,
             float(scaled.eps) if scaled is not None else 0.0, positions.data_ptr(), token_req.data_ptr(),
             block_table.data_ptr(), block_table.stride(0), inv_freq.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
             int(page_size), nq, nkv, head_dim, inv_freq.numel(), int(bool(write_kv)), _tc(xt.device).error.data_ptr(), _stream())
    return True


GATE_BLOCK = 64  # gate and up rows alternate in runs of this many in a packed projection that the fused kernel takes


def gated_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, block: int) -> torch.Tensor:
    """out[n, j] = silu(x @ gate_j) * (x @ up_j) for a packed projection w [2I, K]: [gate | up] when
    `block` is 0, runs of `block` gate rows followed by the matching up rows otherwise.  A decode step
    in bfloat16 with block == GATE_BLOCK is one tcgen05 kernel whose epilogue applies the activation;
    everything else is the product into `scratch` [N, 2I] and the swiglu kernel.  `x` may be a `RowScaled`."""
    if isinstance(x, RowScaled):
        if block == GATE_BLOCK and out.dtype == torch.bfloat16:
            return _linear_norm(x, w, out, True, None)
        return swiglu(_linear_norm(x, w, scratch, False, None), out, block)
    _cuda(x, w, out, scratch)
    M, K = x.shape
    if x.dtype == torch.bfloat16 and block == GATE_BLOCK and USE_TENSOR_CORE_GEMM and w.shape[0] % 128 == 0 \
            and TENSOR_CORE_GEMM_MAX_TOKENS is not None and M <= TENSOR_CORE_GEMM_MAX_TOKENS \
            and out.dtype == torch.bfloat16 and not (K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16
                                                     or w.data_ptr() % 16 or x.stride(1) != 1 or w.stride(1) != 1):
        if w.shape[1] != K or out.shape != (M, w.shape[0] // 2) or out.stride(1) != 1:
            raise KernelError(f"gated_linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
        lib.call("ns_gemm_bf16_tc_gated", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, w.shape[0], K, x.stride(0),
                 w.stride(0), out.stride(0), 0, gemm_splits(M, w.shape[0], K), _tc(x.device).error.data_ptr(), _stream())
        return out
    return swiglu(linear(x, w, scratch), out, block)


def attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      token_req: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, nq: int, nkv: int,
                      head_dim: int, page_size: int, scale: float | None = None, window: int = 0) -> torch.Tensor:
    """q: [N, >= nq*head_dim] rows (a view into the packed projection is fine, unit inner
    stride); out: [N, nq*head_dim].  See csrc/attention_generic.cu for the masking rule."""
    _cuda(q, k_cache, v_cache, block_table, token_req, positions, out)
    _i32(positions, "positions"), _i32(token_req, "token_req")
    n = out.shape[0]
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[0] != n or q.dtype != out.dtype:
        raise KernelError("attention: q and out must be row-major with the same rows and dtype")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise KernelError("attention: the cache must hold the activations' dtype")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    lib.call("ns_attention_generic", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
             block_table.data_ptr(), block_table.stride(0), token_req.data_ptr(), positions.data_ptr(),
             out.data_ptr(), out.stride(0), n, nq, nkv, head_dim, page_size, float(scale), int(window),
             dtype_code(q.dtype), _stream())
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                u: torch.Tensor, out: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
                scratch: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per row of fp32 logits: (token int32, raw log-prob, processed log-prob); `out` gives
    preallocated result tensors (int32, float32, float32, one entry per row) and `scratch` a
    preallocated float32 buffer of 48 floats per row for the kernel's first pass."""
    _cuda(logits, temperature, top_k, top_p, u)
    _i32(top_k, "top_k")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample_rows: logits must be float32 rows")
    for t, name in ((temperature, "temperature"), (top_p, "top_p"), (u, "u")):
        if t.dtype != torch.float32 or t.numel() != rows or not t.is_contiguous():
            raise KernelError(f"sample_rows: {name} must be one contiguous float32 per row")
    if out is not None:
        token, lp_raw, lp_proc = out
        if token.dtype != torch.int32 or lp_raw.dtype != torch.float32 or lp_proc.dtype != torch.float32 \
                or min(token.numel(), lp_raw.numel(), lp_proc.numel()) < rows:
            raise KernelError("sample_rows: out must be (int32, float32, float32) with one entry per row")
    else:
        token = torch.empty(rows, dtype=torch.int32, device=logits.device)
        lp_raw = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lp_proc = torch.empty(rows, dtype=torch.float32, device=logits.device)
    if scratch is None:
        scratch = torch.empty(rows * 48, dtype=torch.float32, device=logits.device)
    elif scratch.dtype != torch.float32 or scratch.numel() < rows * 48 or not scratch.is_contiguous():
        raise KernelError("sample_rows: scratch must be contiguous float32 with 48 entries per row")
    lib.call("ns_sample_rows", logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(),
             top_k.data_ptr(), top_p.data_ptr(), u.data_ptr(), scratch.data_ptr(), token.data_ptr(), lp_raw.data_ptr(),
             lp_proc.data_ptr(), _stream())
    return token, lp_raw, lp_proc


def kv_store(qkv: torch.Tensor, ctx, lane, nq: int, nkv: int, head_dim: int) -> None:
    """Stores k and v of the packed projection at each token's cache slot, unrotated."""
    none = torch.empty(0, dtype=torch.float32, device=qkv.device)
    rope_kv_write(qkv, ctx.positions, ctx.token_req, lane.block_table, none, lane.k, lane.v, lane.page_size, nq, nkv,
                  head_dim, write_kv=True)


TILE_Q = 128         # query rows per block of the m16n8k16 prefill kernel
TILE_Q_TCGEN05 = 256 # and of the tcgen05 one (two tiles of 128)
USE_TCGEN05_ATTENTION = True


def _target_blocks() -> int:
    """Decode attention wants about two blocks per SM before it splits keys further."""
    return 2 * sm_count()


def _tensor_core_attention(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128


USE_CLUSTER_DECODE = True


def _cluster_decode_splits(blocks: int, max_kv_len: int | None) -> int:
    """Blocks of one cluster that share a request's keys: a power of two up to 16 that keeps the grid
    within two blocks per SM (measured on a B200: 16 at one request, 4 at 8, 1 at 64, for contexts of
    1,024 and 4,096), and, when the longest context is known, at least two tiles of 64 keys per block."""
    n_splits = 1
    while n_splits < 16 and blocks * n_splits * 2 <= _target_blocks():
        n_splits *= 2
    if max_kv_len is not None:
        while n_splits > 1 and max_kv_len < 128 * n_splits:
            n_splits //= 2
    return n_splits


def attention_decode(qkv: torch.Tensor, lane, ctx, out: torch.Tensor, nq: int, nkv: int, head_dim: int, scale: float,
                     window: int, rows: torch.Tensor | None, n_rows: int, max_kv_len: int | None,
                     work: torch.Tensor | None = None, work_slots: int = 0) -> None:
    """Split-KV decode attention for the requests that bring one token.  Head sizes 64 and 128 with
    pages of 8 to 64 tokens: TMA loads and a thread-block cluster per request and kv head
    (csrc/attention_decode_tma.cu); everything else: cp.async loads and a merge through global
    memory (csrc/attention_decode.cu).
    `rows`: int32 device tensor of their token rows, or None when every row of the step is one.
    `work` (int32, four per item, from the cache manager's packer) replaces `rows` for the TMA kernel on lanes without
    a window: a request whose context is much longer than the others' comes as several items, a part of its keys
    each, and the kernel adds the parts up through `work_slots` slots of scratch."""
    head_tiles = -(-(nq // nkv) // 16)
    if USE_CLUSTER_DECODE and head_dim in (64, 128) and lane.page_size in (8, 16, 32, 64) and qkv.stride(0) % 2 == 0:
        n_splits = _cluster_decode_splits(n_rows * nkv * head_tiles, max_kv_len)
        if work is not None and window == 0:
            ws = ctx.workspace
            part = ws.get("attn_work_parts", max(work_slots, 1) * nkv * head_tiles, 16 * head_dim + 32, torch.float32)
            counters = ws.get("attn_work_counters", max(work_slots, 1) * nkv * head_tiles, 1, torch.int32, zero=True)
            lib.call("ns_attention_decode_tma", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
                     lane.k.shape[0], lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.token_req.data_ptr(),
                     ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(), out.data_ptr(), out.stride(0), None,
                     work.numel() // 4, nq, nkv, head_dim, lane.page_size, float(scale), 0, n_splits,
                     _tc(qkv.device).error.data_ptr(), work.data_ptr(), part.data_ptr(), counters.data_ptr(), _stream())
            return
        lib.call("ns_attention_decode_tma", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
                 lane.k.shape[0], lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.token_req.data_ptr(),
                 ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(), out.data_ptr(), out.stride(0), _ptr(rows), n_rows, nq,
                 nkv, head_dim, lane.page_size, float(scale), int(window), n_splits, _tc(qkv.device).error.data_ptr(),
                 None, None, None, _stream())
        return
    n_splits = max(1, min(16, -(-_target_blocks() // (n_rows * nkv * head_tiles))))
    if max_kv_len is not None:
        # long contexts split further (measured: 4 splits are best at 4,096 keys even for 64 requests),
        # and a split keeps at least two tiles of keys
        n_splits = max(n_splits, min(4, max_kv_len // 1024))
        n_splits = max(1, min(n_splits, -(-max_kv_len // 128)))
    ws = ctx.workspace
    part_o = ws.get("attn_part_o", n_rows * nq * n_splits, head_dim, torch.float32)
    part_ml = ws.get("attn_part_ml", n_rows * nq * n_splits, 2, torch.float32)
    counters = ws.get("attn_counters", n_rows * nkv * head_tiles, 1, torch.int32, zero=True)
    lib.call("ns_attention_decode", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
             lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.token_req.data_ptr(), ctx.positions.data_ptr(),
             ctx.qo_indptr.data_ptr(), out.data_ptr(), out.stride(0), part_o.data_ptr(), part_ml.data_ptr(),
             counters.data_ptr(), _ptr(rows), n_rows, nq, nkv, head_dim, lane.page_size, float(scale), int(window),
             n_splits, _stream())


PREFILL_TWO_HEADS = "auto"  # "always" / "never": tests run both kernels whatever the size of the grid


def attention_prefill(qkv: torch.Tensor, lane, ctx, out: torch.Tensor, nq: int, nkv: int, head_dim: int, scale: float,
                      window: int, tiles: torch.Tensor, tiles_tc: torch.Tensor | None = None) -> None:
    """Tensor-core attention for portions of prompts.  `tiles`: int32 [n, 2] of (request, offset
    among its tokens of this step).  Head sizes 64 and 128 with pages of 8 to 64 tokens and no window run
    on tcgen05 (csrc/attention_prefill_tc.cu); everything else on m16n8k16 (csrc/attention_prefill.cu)."""
    if USE_TCGEN05_ATTENTION and tiles_tc is not None and head_dim in (64, 128) and window == 0 \
            and lane.page_size in (8, 16, 32, 64) and qkv.stride(0) % 8 == 0 and out.stride(0) % 8 == 0:
        # heads of 64: two query heads of a kv head to a block (four softmax warps per sub-partition keep the exponential
        # unit busier and the keys are read once for both) - once one head to a block would give more blocks than SMs
        two_heads = head_dim == 64 and (nq // nkv) % 2 == 0 and PREFILL_TWO_HEADS != "never" and (
            PREFILL_TWO_HEADS == "always" or nq * tiles_tc.shape[0] > sm_count())
        lib.call("ns_attention_prefill_tc", qkv.data_ptr(), qkv.stride(0), qkv.shape[0], lane.k.data_ptr(),
                 lane.v.data_ptr(), lane.k.shape[0], lane.block_table.data_ptr(), lane.block_table.stride(0),
                 ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(), tiles_tc.data_ptr(), tiles_tc.shape[0], out.data_ptr(),
                 out.stride(0), nq, nkv, head_dim, lane.page_size, float(scale), 2 if two_heads else 1,
                 _tc(qkv.device).error.data_ptr(), _stream())
        return
    lib.call("ns_attention_prefill", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
             lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(),
             tiles.data_ptr(), tiles.shape[0], out.data_ptr(), out.stride(0), nq, nkv, head_dim, lane.page_size,
             float(scale), int(window), _stream())


def _attention_plan(ctx) -> dict:
    """Once per step: which token rows decode, and the query tiles of the prompt portions."""
    plan = ctx.extras.get("attention_plan")
    if plan is not None:
        return plan
    if ctx.extras.get("graph"):
        plan = {"decode_rows": None, "n_decode": ctx.n_tokens, "tiles": None, "tiles_tc": None, "max_kv_len": None}
    else:
        starts, row = [], 0
        for n in ctx.q_lens:
            starts.append(row)
            row += n
        decode = [s for s, n in zip(starts, ctx.q_lens) if n == 1]
        # the tiles that see the most keys come first: blocks are scheduled in this order
        def make(tile_q):
            ts = [(b, off) for b, n in enumerate(ctx.q_lens) if n > 1 for off in range(0, n, tile_q)]
            ts.sort(key=lambda t: -(ctx.kv_lens[t[0]] - ctx.q_lens[t[0]] + min(t[1] + tile_q, ctx.q_lens[t[0]])))
            return ts
        tiles, tiles_tc = make(TILE_Q), make(TILE_Q_TCGEN05)
        dev = ctx.device
        plan = {
            "n_decode": len(decode),
            "decode_rows": None if len(decode) == ctx.n_tokens or not decode
            else torch.tensor(decode, dtype=torch.int32).to(dev, non_blocking=True),
            "tiles": torch.tensor(tiles, dtype=torch.int32).to(dev, non_blocking=True) if tiles else None,
            "tiles_tc": torch.tensor(tiles_tc, dtype=torch.int32).to(dev, non_blocking=True) if tiles_tc else None,
            "max_kv_len": max((kv for kv, n in zip(ctx.kv_lens, ctx.q_lens) if n == 1), default=None),
        }
    ctx.extras["attention_plan"] = plan
    return plan


def attention(qkv: torch.Tensor, lane, ctx, out: torch.Tensor, nq: int, nkv: int, head_dim: int, scale: float,
              window: int = 0) -> torch.Tensor:
    """Attention of the step's queries (the first nq*head_dim columns of `qkv`) over `lane`.

    bfloat16 with a head size that the tensor-core kernels take: the decode kernel for requests
    that bring one token, the prefill kernel for the others.  float32, and head sizes those
    kernels refuse: the exact kernel, one warp per (token, head)."""
    if not _tensor_core_attention(qkv.dtype, head_dim) or nq // nkv > 64:
        return attention_generic(qkv, lane.k, lane.v, lane.block_table, ctx.token_req, ctx.positions, out, nq, nkv,
                                 head_dim, lane.page_size, scale, window)
    _cuda(qkv, out, lane.k, lane.v, lane.block_table)
    if out.stride(1) != 1 or qkv.stride(1) != 1 or lane.k.dtype != qkv.dtype:
        raise KernelError("attention: row-major bfloat16 operands and a bfloat16 cache are needed")
    plan = _attention_plan(ctx)
    both = bool(plan["n_decode"]) and plan["tiles"] is not None
    if both and OVERLAP_MIXED_ATTENTION and not torch.cuda.is_current_stream_capturing():
        # A step of decode tokens beside portions of prompts: the two kernels read the same cache and write different rows.
        # The decode kernel goes to a side stream, so that its blocks fill the SMs which the prefill kernel's last,
        # ragged round of blocks leaves idle instead of running before it on an otherwise empty GPU.
        main = torch.cuda.current_stream()
        side = _side_stream(qkv.device)
        fork, join = _side_events(qkv.device)
        fork.record(main)
        side.wait_event(fork)
        attention_prefill(qkv, lane, ctx, out, nq, nkv, head_dim, scale, window, plan["tiles"], plan.get("tiles_tc"))
        with torch.cuda.stream(side):
            attention_decode(qkv, lane, ctx, out, nq, nkv, head_dim, scale, window, plan["decode_rows"], plan["n_decode"],
                             plan["max_kv_len"], plan.get("work"), plan.get("work_slots", 0))
            join.record(side)
        main.wait_event(join)
        return out
    if plan["n_decode"]:
        attention_decode(qkv, lane, ctx, out, nq, nkv, head_dim, scale, window, plan["decode_rows"], plan["n_decode"],
                         plan["max_kv_len"], plan.get("work"), plan.get("work_slots", 0))
    if plan["tiles"] is not None:
        attention_prefill(qkv, lane, ctx, out, nq, nkv, head_dim, scale, window, plan["tiles"], plan.get("tiles_tc"))
    return out


OVERLAP_MIXED_ATTENTION = True
_side: dict = {}


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    st = _side.get((device, "stream"))
    if st is None:
        st = _side[(device, "stream")] = torch.cuda.Stream(device=device)
    return st


def _side_events(device: torch.device):
    ev = _side.get((device, "events"))
    if ev is None:
        ev = _side[(device, "events")] = (torch.cuda.Event(), torch.cuda.Event())
    return ev


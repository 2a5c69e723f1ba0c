"""Each CUDA kernel alone against a plain float32 PyTorch statement of the same operation,
at sizes other than the engine's tiny models use: widths and vocabularies that are no power
of two, head sizes in steps of 16, odd group counts, scattered pages.  Where random inputs
would hide a fault the inputs are made so that it shows (one far key that dominates, a
window's edge, a key on a page boundary)."""

from __future__ import annotations

import math

import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from nanospec_b200 import ops as o
    return o


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,vocab", [(100, 77), (4096, 300), (1536, 1000)])
def test_embed(dtype, hidden, vocab):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, hidden, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (37,), generator=g).to(torch.int32)
    ids[5] = -1  # a padding row
    out = torch.full((37, hidden), 7.0, device=DEV)
    ops().embed(table, ids.to(DEV), out)
    want = table.float()[ids.clamp(min=0).long().to(DEV)]
    want[5] = 0
    assert torch.equal(out, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [64, 100, 1000, 4096, 5000, 9001])
def test_add_rmsnorm(dtype, hidden):
    g = torch.Generator().manual_seed(hidden)
    n = 13
    resid = torch.randn(n, hidden, generator=g).to(DEV) * 3
    branch = torch.randn(n, hidden, generator=g).to(dtype).to(DEV)
    gain = (1 + 0.1 * torch.randn(hidden, generator=g)).to(DEV)
    eps = 1e-3
    want_resid = resid + branch.float()
    want = plain.plain_rmsnorm(want_resid.cpu(), gain.cpu(), eps).to(DEV)
    r = resid.clone()
    out = torch.empty(n, hidden, dtype=dtype, device=DEV)
    ops().add_rmsnorm(r, branch, gain, eps, out)
    assert torch.allclose(r, want_resid, rtol=0, atol=0)
    torch.testing.assert_close(out.float(), want, **tol(dtype))
    # without a branch the residual is untouched
    r2 = resid.clone()
    ops().add_rmsnorm(r2, None, gain, eps, out)
    assert torch.equal(r2, resid)
    torch.testing.assert_close(out.float(), plain.plain_rmsnorm(resid.cpu(), gain.cpu(), eps).to(DEV), **tol(dtype))
    # row selection: only the asked rows, residual untouched even with a branch
    rows = torch.tensor([11, 0, 4], dtype=torch.int32, device=DEV)
    r3 = resid.clone()
    out3 = torch.empty(3, hidden, dtype=dtype, device=DEV)
    ops().add_rmsnorm(r3, branch, gain, eps, out3, rows=rows)
    assert torch.equal(r3, resid)
    torch.testing.assert_close(out3.float(), want[rows.long()], **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_and_residual_add(dtype):
    g = torch.Generator().manual_seed(3)
    n, inter = 9, 352
    gu = (torch.randn(n, 2 * inter, generator=g) * 4).to(dtype).to(DEV)
    out = torch.empty(n, inter, dtype=dtype, device=DEV)
    ops().swiglu(gu, out)
    f = gu.float()
    want = torch.nn.functional.silu(f[:, :inter]) * f[:, inter:]
    torch.testing.assert_close(out.float(), want, **tol(dtype))
    # gate and up alternating in runs of 32 features
    inter2, block = 320, 32
    gu2 = (torch.randn(n, 2 * inter2, generator=g) * 4).to(dtype).to(DEV)
    out2 = torch.empty(n, inter2, dtype=dtype, device=DEV)
    ops().swiglu(gu2, out2, block)
    f2 = gu2.float().view(n, inter2 // block, 2, block)
    want2 = (torch.nn.functional.silu(f2[:, :, 0]) * f2[:, :, 1]).reshape(n, inter2)
    torch.testing.assert_close(out2.float(), want2, **tol(dtype))
    resid = torch.randn(n, inter, generator=g).to(DEV)
    want_r = resid + out.float()
    ops().residual_add(resid, out)
    assert torch.equal(resid, want_r)


@pytest.mark.parametrize("M,N,K", [(1, 70, 33), (3, 64, 64), (130, 257, 100), (65, 331, 96), (7, 512, 353)])
def test_gemm_f32_is_true_fp32_and_independent_of_m(M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).to(DEV)
    w = torch.randn(N, K, generator=g).to(DEV)
    out = torch.empty(M, N, device=DEV)
    ops().linear(x, w, out)
    want = (x.double() @ w.double().T)
    err = (out.double() - want).abs().max().item()
    assert err < 1e-5 * math.sqrt(K) * 4, err  # fp32 rounding only; TF32 would be ~1e-3
    # each row alone gives the very same bits as the row inside the batch
    for m in {0, M // 2, M - 1}:
        one = torch.empty(1, N, device=DEV)
        ops().linear(x[m:m + 1].contiguous(), w, one)
        assert torch.equal(one[0], out[m])


def paged(k: torch.Tensor, v: torch.Tensor, page: int, n_pages: int, seed: int):
    """Scatters contiguous k, v [S, nkv, d] over randomly chosen pages; returns the page
    tensors and the block table row."""
    S, nkv, d = k.shape
    g = torch.Generator().manual_seed(seed)
    nb = -(-S // page)
    pages = torch.randperm(n_pages, generator=g)[:nb]
    kc = torch.zeros(n_pages, nkv, page, d, dtype=k.dtype)  # cache[page, kv head, offset, :]
    vc = torch.zeros(n_pages, nkv, page, d, dtype=k.dtype)
    for b in range(nb):
        lo, hi = b * page, min(S, (b + 1) * page)
        kc[pages[b], :, : hi - lo] = k[lo:hi].transpose(0, 1)
        vc[pages[b], :, : hi - lo] = v[lo:hi].transpose(0, 1)
    return kc, vc, pages.to(torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lens", [[7, 12], [90, 33]])  # few tokens: a block per (token, head); many: a block per token
@pytest.mark.parametrize("nq,nkv,d,page", [(6, 3, 16, 4), (8, 2, 64, 16), (5, 5, 48, 8), (4, 1, 128, 16)])
def test_rope_kv_write(dtype, nq, nkv, d, page, lens):
    g = torch.Generator().manual_seed(d)
    n_pages = 240
    scaling = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    inv = plain.plain_inv_freq(d, 500000.0, scaling)
    # two requests: one continues at a late position (large angles), one starts at 0
    starts = [301, 0]
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    tables_big = torch.stack([perm[:120], perm[120:]])  # disjoint, scattered pages for every logical block
    positions, token_req = [], []
    for r, (s, n) in enumerate(zip(starts, lens)):
        positions += list(range(s, s + n))
        token_req += [r] * n
    positions.insert(3, 0), token_req.insert(3, -1)  # a padding row in the middle
    N = len(positions)
    qkv = torch.randn(N, (nq + 2 * nkv) * d, generator=g).to(dtype)
    kc = torch.zeros(n_pages, nkv, page, d, dtype=dtype, device=DEV)  # cache[page, kv head, offset, :]
    vc = torch.zeros_like(kc)
    dev_qkv = qkv.clone().to(DEV)
    ops().rope_kv_write(dev_qkv, torch.tensor(positions, dtype=torch.int32, device=DEV),
                        torch.tensor(token_req, dtype=torch.int32, device=DEV), tables_big.to(DEV), inv.to(DEV), kc, vc,
                        page, nq, nkv, d)
    f = qkv.float()
    pos_t = torch.tensor(positions)
    q_want = plain.plain_rope(f[:, : nq * d].view(N, nq, d), pos_t, inv)
    k_want = plain.plain_rope(f[:, nq * d: (nq + nkv) * d].view(N, nkv, d), pos_t, inv)
    v_in = f[:, (nq + nkv) * d:].view(N, nkv, d)
    got = dev_qkv.float().cpu()
    for n in range(N):
        if token_req[n] < 0:
            assert torch.equal(got[n], f[n])  # padding rows are left alone
            continue
        torch.testing.assert_close(got[n, : nq * d].view(nq, d), q_want[n], **tol(dtype))
        pg = int(tables_big[token_req[n], positions[n] // page])
        off = positions[n] % page
        torch.testing.assert_close(kc[pg, :, off].float().cpu(), k_want[n], **tol(dtype))
        assert torch.equal(vc[pg, :, off].float().cpu(), v_in[n])
        # v and the unrotated part of the row stay as they were
        assert torch.equal(got[n, nq * d:], f[n, nq * d:])
    assert int((kc != 0).any(dim=-1).any(dim=1).sum()) == sum(lens)  # nothing else was written


def attention_case(dtype, nq, nkv, d, page, S, window, spike_key=None, seed=0):
    """One request of S positions; the last `q_len` are this step's queries."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(S, nq, d, generator=g)
    k = torch.randn(S, nkv, d, generator=g)
    v = torch.randn(S, nkv, d, generator=g)
    if spike_key is not None:
        # one far key that every query must find: scale it and align the queries with it
        k[spike_key] = 4.0 * k[spike_key] / k[spike_key].norm(dim=-1, keepdim=True) * math.sqrt(d)
        q = q + 0.75 * k[spike_key].repeat_interleave(nq // nkv, dim=0)[None]
        v[spike_key] = 10.0
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    want = plain.plain_attention(q.float(), k.float(), v.float(), window=window)
    return q, k, v, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,page,S,window,spike", [
    (6, 3, 16, 4, 70, 0, None),
    (8, 2, 64, 16, 300, 0, 3),       # a far key among hundreds
    (4, 1, 128, 16, 257, 0, 255),    # the key just before a page edge
    (12, 4, 80, 8, 150, 0, 64),      # head size in steps of 16, key on a page's first slot
    (5, 5, 48, 8, 130, 17, 100),     # window whose edge falls inside a page
    (8, 8, 32, 16, 96, 32, 64),      # window edge on a page edge: key 64 is the first visible to query 95
    (2, 1, 256, 16, 40, 0, None),
    (7, 7, 8, 16, 50, 0, 1),
])
def test_attention_generic(dtype, nq, nkv, d, page, S, window, spike):
    q, k, v, want = attention_case(dtype, nq, nkv, d, page, S, window, spike, seed=S)
    n_pages = 2 * (-(-S // page)) + 3
    kc, vc, table = paged(k, v, page, n_pages, seed=S + 1)
    for q_len in (1, 2, S // 3, S):  # decode, a two-token portion, a portion in the middle, the whole
        start = S - q_len
        positions = torch.arange(start, S, dtype=torch.int32, device=DEV)
        token_req = torch.zeros(q_len, dtype=torch.int32, device=DEV)
        # q sits inside a wider row, as in the packed projection
        qrow = torch.zeros(q_len, (nq + 2 * nkv) * d, dtype=dtype)
        qrow[:, : nq * d] = q[start:].reshape(q_len, nq * d)
        out = torch.empty(q_len, nq * d, dtype=dtype, device=DEV)
        ops().attention_generic(qrow.to(DEV), kc.to(DEV), vc.to(DEV), table[None].to(DEV), token_req, positions, out,
                                nq, nkv, d, page, None, window)
        torch.testing.assert_close(out.float().cpu().view(q_len, nq, d), want[start:],
                                   **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)))


def test_attention_generic_batch_of_requests_and_padding():
    dtype = torch.float32
    nq, nkv, d, page = 4, 2, 32, 8
    cases = [attention_case(dtype, nq, nkv, d, page, S, 0, spike, seed=S) for S, spike in ((33, 2), (8, None), (100, 50))]
    n_pages = 64
    kc = torch.zeros(n_pages, nkv, page, d)
    vc = torch.zeros_like(kc)
    tables = torch.zeros(3, 16, dtype=torch.int32)
    free = list(torch.randperm(n_pages, generator=torch.Generator().manual_seed(5)).tolist())
    for r, (q, k, v, _) in enumerate(cases):
        S = k.shape[0]
        for b in range(-(-S // page)):
            pg = free.pop()
            tables[r, b] = pg
            lo, hi = b * page, min(S, (b + 1) * page)
            kc[pg, :, : hi - lo], vc[pg, :, : hi - lo] = k[lo:hi].transpose(0, 1), v[lo:hi].transpose(0, 1)
    q_lens = [1, 8, 13]
    rows, positions, token_req, want = [], [], [], []
    for r, ((q, k, v, w), n) in enumerate(zip(cases, q_lens)):
        S = k.shape[0]
        rows.append(q[S - n:].reshape(n, nq * d))
        want.append(w[S - n:])
        positions += list(range(S - n, S))
        token_req += [r] * n
    qrows = torch.cat(rows)
    # a padding row at the end
    qrows = torch.cat([qrows, torch.zeros(1, nq * d)])
    positions.append(0), token_req.append(-1)
    out = torch.full((qrows.shape[0], nq * d), 5.0, device=DEV)
    ops().attention_generic(qrows.to(DEV), kc.to(DEV), vc.to(DEV), tables.to(DEV),
                            torch.tensor(token_req, dtype=torch.int32, device=DEV),
                            torch.tensor(positions, dtype=torch.int32, device=DEV), out, nq, nkv, d, page)
    torch.testing.assert_close(out[:-1].cpu().view(-1, nq, d), torch.cat(want), rtol=1e-4, atol=1e-5)
    assert torch.equal(out[-1].cpu(), torch.full((nq * d,), 5.0))  # padding row untouched


@pytest.mark.parametrize("vocab", [331, 1000, 128256])
def test_sample_rows(vocab):
    g = torch.Generator().manual_seed(vocab)
    rows = 12
    z = torch.randn(rows, vocab, generator=g) * 2.5
    z[0, 17] = z[0, 200] = z[0].max() + 1.0  # a tie for the maximum: the lowest index wins
    temps = [0.0, 0.0, 0.8, 1.0, 1.3, 0.7, 1.0, 0.5, 1.0, 2.0, 0.9, 1.0]
    top_k = [0, 0, 0, 0, 5, 0, 7, 50, 1, 0, vocab + 5, 3]
    top_p = [1.0, 1.0, 1.0, 1.0, 1.0, 0.6, 0.9, 0.95, 1.0, 0.3, 1.0, 0.0]
    us = torch.rand(rows, generator=g).tolist()
    us[3] = 0.999999
    tok, lp_raw, lp_proc = ops().sample_rows(
        z.to(DEV), torch.tensor(temps, device=DEV), torch.tensor(top_k, dtype=torch.int32, device=DEV),
        torch.tensor(top_p, device=DEV), torch.tensor(us, device=DEV))
    tok, lp_raw, lp_proc = tok.cpu().tolist(), lp_raw.cpu(), lp_proc.cpu()
    lse = z.logsumexp(-1)
    for r in range(rows):
        if temps[r] == 0:
            want = int(z[r].argmax()) if r else 17
            assert tok[r] == want and lp_proc[r] == 0
        else:
            lp = plain.plain_process(z[r], temps[r], top_k[r], top_p[r])
            want = plain.plain_draw(lp, us[r])
            if tok[r] != want:
                # an inverse-CDF draw may flip at a boundary of the cdf under another order of sums
                cdf = lp.exp().cumsum(-1)
                target = us[r] * cdf[-1]
                near = min(abs(float(cdf[min(tok[r], want)] - target)), abs(float(cdf[max(tok[r], want) - 1] - target)))
                assert abs(tok[r] - want) >= 1 and near < 1e-5, (r, tok[r], want, near)
            assert torch.isfinite(lp[tok[r]]), f"row {r}: token {tok[r]} lies outside the kept set"
            assert abs(float(lp_proc[r]) - float(lp[tok[r]])) < 1e-4
        assert abs(float(lp_raw[r]) - float(z[r, tok[r]] - lse[r])) < 1e-4


# ---------------------------------------------------------------------------------------
# the bfloat16 tensor-core attention kernels (decode: split-KV; prefill: 64-query tiles)
# ---------------------------------------------------------------------------------------
def _step(requests, nq, nkv, d, page, n_pages, seed):
    """requests: list of (S, q_len, spike).  Builds one paged cache for all of them and the
    flattened step; returns (ctx, lane, qkv rows, expected outputs per request)."""
    from types import SimpleNamespace
    from nanospec_b200.parts import Workspace
    kc = torch.zeros(n_pages, nkv, page, d, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    free = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max(-(-S // page) for S, _, _ in requests)
    tables = torch.zeros(len(requests), width, dtype=torch.int32)
    rows, positions, token_req, qo, want, windows = [], [], [], [0], [], None
    for r, (S, q_len, spike) in enumerate(requests):
        q, k, v, _ = attention_case(torch.bfloat16, nq, nkv, d, page, S, 0, spike, seed=seed + 7 * r)
        for b in range(-(-S // page)):
            pg = free.pop()
            tables[r, b] = pg
            lo, hi = b * page, min(S, (b + 1) * page)
            kc[pg, :, : hi - lo], vc[pg, :, : hi - lo] = k[lo:hi].transpose(0, 1), v[lo:hi].transpose(0, 1)
        rows.append(q[S - q_len:].reshape(q_len, nq * d))
        positions += list(range(S - q_len, S))
        token_req += [r] * q_len
        qo.append(qo[-1] + q_len)
        want.append((q.float(), k.float(), v.float(), S - q_len))
    N = len(positions)
    qkv = torch.zeros(N, (nq + 2 * nkv) * d, dtype=torch.bfloat16)
    qkv[:, : nq * d] = torch.cat(rows)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(n_tokens=N, token_req=i32(token_req), positions=i32(positions), qo_indptr=i32(qo),
                          q_lens=[q for _, q, _ in requests], kv_lens=[S for S, _, _ in requests], device=torch.device(DEV),
                          extras={}, workspace=Workspace(torch.device(DEV)), max_q_len=max(q for _, q, _ in requests))
    lane = SimpleNamespace(k=kc.to(DEV), v=vc.to(DEV), block_table=tables.to(DEV), page_size=page)
    return ctx, lane, qkv.to(DEV), want


@pytest.mark.parametrize("nq,nkv,d,page,window", [
    (8, 2, 128, 16, 0), (4, 1, 32, 8, 0), (6, 3, 16, 4, 0), (12, 4, 80, 16, 0), (5, 5, 48, 8, 0), (32, 8, 64, 16, 0),
    (8, 2, 64, 16, 100), (4, 4, 112, 8, 64), (40, 2, 32, 16, 0),
])
def test_tensor_core_attention_mixed_step(nq, nkv, d, page, window):
    """Decode rows beside portions of prompts in one step: (S, q_len, far key that must be found)."""
    requests = [(700, 1, 3), (65, 1, 64), (130, 130, 5), (333, 70, 2), (64, 2, 63), (1, 1, None), (257, 129, 128), (90, 1, None)]
    ctx, lane, qkv, want = _step(requests, nq, nkv, d, page, n_pages=2000 // page + 40, seed=d + nq)
    out = torch.zeros(ctx.n_tokens, nq * d, dtype=torch.bfloat16, device=DEV)
    ops().attention(qkv, lane, ctx, out, nq, nkv, d, 1.0 / math.sqrt(d), window)
    assert ctx.extras["attention_plan"]["n_decode"] == 4 and ctx.extras["attention_plan"]["tiles"].shape[0] == 2 + 1 + 1 + 2
    row = 0
    for (S, q_len, _), (q, k, v, start) in zip(requests, want):
        full = plain.plain_attention(q, k, v, window=window)
        torch.testing.assert_close(out[row: row + q_len].float().cpu().view(q_len, nq, d), full[start:], rtol=3e-2, atol=3e-2)
        row += q_len


@pytest.mark.parametrize("n_req,S", [(1, 1500), (3, 1030), (64, 70)])
def test_decode_attention_splits_and_counters(n_req, S):
    """Decode only, long enough that the keys are split over several blocks; run twice on the same
    scratch (the counters must come back to zero) and in the layout a captured graph uses."""
    nq, nkv, d, page = 8, 2, 128, 16
    requests = [(S - 13 * (r % 5), 1, (S - 13 * (r % 5)) // 2) for r in range(n_req)]
    ctx, lane, qkv, want = _step(requests, nq, nkv, d, page, n_pages=n_req * (S // page + 2), seed=S)
    for cluster in (True, False):  # the TMA kernel with its cluster, and the cp.async kernel with its counters
        ops().USE_CLUSTER_DECODE = cluster
        for graph in (False, True):
            ctx.extras = {"graph": True} if graph else {}
            for _ in range(2):
                out = torch.zeros(ctx.n_tokens, nq * d, dtype=torch.bfloat16, device=DEV)
                ops().attention(qkv, lane, ctx, out, nq, nkv, d, 1.0 / math.sqrt(d), 0)
                for r, (q, k, v, start) in enumerate(want):
                    full = plain.plain_attention(q, k, v)
                    torch.testing.assert_close(out[r].float().cpu().view(nq, d), full[start], rtol=3e-2, atol=3e-2)
    ops().USE_CLUSTER_DECODE = True
    ops().check_kernel_errors()
    assert int(ctx.workspace.get("attn_counters", 1, 1, torch.int32).sum()) == 0


@pytest.mark.parametrize("nq,nkv,d,page,window", [(8, 2, 128, 16, 0), (4, 4, 64, 8, 0), (6, 1, 128, 32, 200), (40, 2, 64, 64, 0),
                                                  (32, 8, 128, 64, 0), (8, 2, 128, 8, 70)])
def test_cluster_decode_attention(nq, nkv, d, page, window):
    """The TMA decode kernel alone, at every cluster size: contexts from one key to a few thousand, a far key
    that must be found, a window whose first page is not the tile's first, rows picked out of a larger
    step, twice in a row - against the plain attention."""
    lens = [1, 5, 63, 64, 65, 130, 1000, 2100, 777]
    requests = [(S, 1, S // 2 if S > 4 else None) for S in lens] + [(300, 40, 7)]  # the last one is not a decode row
    ctx, lane, qkv, want = _step(requests, nq, nkv, d, page, n_pages=sum(-(-S // page) for S in lens) + 40, seed=d + page)
    rows = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    o, lib = ops(), ops().lib
    err = o._tc(torch.device(DEV)).error
    for n_splits in (1, 2, 4, 8, 16):
        for _ in range(2):
            out = torch.zeros(ctx.n_tokens, nq * d, dtype=torch.bfloat16, device=DEV)
            lib.call("ns_attention_decode_tma", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
                     lane.k.shape[0], lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.token_req.data_ptr(),
                     ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(), out.data_ptr(), out.stride(0), rows.data_ptr(),
                     len(lens), nq, nkv, d, page, 1.0 / math.sqrt(d), window, n_splits, err.data_ptr(), None, None, None,
                     torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            o.check_kernel_errors()
            for r, (q, k, v, start) in enumerate(want[:-1]):
                full = plain.plain_attention(q, k, v, window=window)
                torch.testing.assert_close(out[r].float().cpu().view(nq, d), full[start], rtol=3e-2, atol=3e-2)
            assert float(out[len(lens):].abs().sum()) == 0.0  # the prompt portion's rows are not touched
    if window:
        return
    # The same rows through a work list in which the long requests come in parts (two, five, and three of which the last
    # holds two keys), an unused item sits in the middle, and the items are not in row order: the parts are added up
    # by whichever block finishes last, and the counters are left at zero for the next launch.
    items, slot = [], 0
    cuts = {6: 2, 7: 5, 5: 3}
    for r, S in enumerate(lens):
        if r in cuts:
            for c in range(cuts[r]):
                items.append((r, r, S, (slot << 8) | (c << 4) | cuts[r]))
            slot += cuts[r]
        else:
            items.append((r, r, S, -1))
    items.insert(3, (-1, -1, 0, -1))
    items = items[::-1]
    work = torch.tensor(items, dtype=torch.int32, device=DEV).contiguous()
    head_tiles = -(-(nq // nkv) // 16)
    part = torch.full((slot * nkv * head_tiles, 16 * d + 32), float("nan"), dtype=torch.float32, device=DEV)
    counters = torch.zeros(slot * nkv * head_tiles, dtype=torch.int32, device=DEV)
    for n_splits in (1, 2, 4, 16):
        for _ in range(2):
            out = torch.zeros(ctx.n_tokens, nq * d, dtype=torch.bfloat16, device=DEV)
            lib.call("ns_attention_decode_tma", qkv.data_ptr(), qkv.stride(0), lane.k.data_ptr(), lane.v.data_ptr(),
                     lane.k.shape[0], lane.block_table.data_ptr(), lane.block_table.stride(0), ctx.token_req.data_ptr(),
                     ctx.positions.data_ptr(), ctx.qo_indptr.data_ptr(), out.data_ptr(), out.stride(0), None,
                     len(items), nq, nkv, d, page, 1.0 / math.sqrt(d), 0, n_splits, err.data_ptr(), work.data_ptr(),
                     part.data_ptr(), counters.data_ptr(), torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            o.check_kernel_errors()
            assert int(counters.abs().sum()) == 0
            for r, (q, k, v, start) in enumerate(want[:-1]):
                full = plain.plain_attention(q, k, v)
                torch.testing.assert_close(out[r].float().cpu().view(nq, d), full[start], rtol=3e-2, atol=3e-2)
            assert float(out[len(lens):].abs().sum()) == 0.0


@pytest.mark.parametrize("nq,nkv,page,d", [(8, 2, 16, 128), (4, 4, 8, 128), (6, 1, 32, 128), (32, 8, 64, 128), (8, 2, 16, 64), (6, 3, 8, 64),
                                           (32, 8, 16, 64), (3, 3, 16, 64), (9, 3, 32, 64), (2, 1, 64, 64)])
def test_tcgen05_prefill_attention(nq, nkv, page, d):
    """Head sizes 64 and 128 take the tcgen05 kernels: prompts from 2 to 1,500 tokens, portions that continue a
    request, tiles that end inside a page, a far key that every query must find - against the plain
    attention and against the m16n8k16 kernel.  Heads of 64 in groups of an even size run two heads to a block
    (four tiles); the same sizes are run once more on the kernel with two tiles that odd groups take."""
    requests = [(1500, 1500, 7), (129, 128, 3), (700, 2, 650), (333, 70, 2), (64, 64, 63), (257, 129, 128), (1000, 300, 640)]
    ctx, lane, qkv, want = _step(requests, nq, nkv, d, page, n_pages=5000 // page + 40, seed=page)
    two_heads = d == 64 and (nq // nkv) % 2 == 0
    outs = {}
    try:
        for tc in (True, False, "one head to a block"):
            if tc == "one head to a block" and not two_heads:
                continue
            ops().USE_TCGEN05_ATTENTION = bool(tc)
            ops().PREFILL_TWO_HEADS = "never" if tc == "one head to a block" else "always"
            ctx.extras = {}
            out = torch.zeros(ctx.n_tokens, nq * d, dtype=torch.bfloat16, device=DEV)
            ops().attention(qkv, lane, ctx, out, nq, nkv, d, 1.0 / math.sqrt(d), 0)
            torch.cuda.synchronize()
            ops().check_kernel_errors()
            outs[tc] = out
    finally:
        ops().USE_TCGEN05_ATTENTION = True
        ops().PREFILL_TWO_HEADS = "auto"
    row = 0
    for (S, q_len, _), (q, k, v, start) in zip(requests, want):
        full = plain.plain_attention(q, k, v)
        for tc in outs:
            torch.testing.assert_close(outs[tc][row: row + q_len].float().cpu().view(q_len, nq, d), full[start:], rtol=3e-2, atol=3e-2)
        row += q_len
    torch.testing.assert_close(outs[True].float(), outs[False].float(), rtol=3e-2, atol=3e-2)
    if two_heads:
        # the same scores in the same blocks of 64 keys: only the lazy reference point may differ between the two
        torch.testing.assert_close(outs["one head to a block"].float(), outs[True].float(), rtol=2e-2, atol=2e-2)

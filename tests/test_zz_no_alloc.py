"""ns_attention_decode_noalloc: decode attention for callers that cannot allocate device
memory (a host whose GPU memory is already in another allocator's hands, a callback in which
allocation is forbidden, a loop that cannot take cudaMalloc's device-wide synchronisation).
Its scratch is a fixed 8 MiB array inside the library instead of caller-provided buffers.

The test calls the entry point through its exported C symbol, twice in a row with different
problems on the shared array, and compares each result with ns_attention_decode given
freshly allocated scratch and with a plain softmax over the keys and values gathered from the
pages (the cache laid out as the kernels read it: [page, kv head, offset, dim]); then checks
that a problem too large for the array is refused with a message that names the limit, and
that one split, which needs no scratch, is never refused for its size.  The file sorts last so that a run that stops at the first
failure has already run every other test."""

from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
NO_ALLOC_BYTES = 8 * 1024 * 1024


def _lib():
    from nanospec_b200.csrc.build import ensure_built
    lib = ctypes.CDLL(str(ensure_built()))
    P, I, F = c_void_p, c_int, c_float
    lib.ns_attention_decode_noalloc.argtypes = [P, I, P, P, P, I, P, P, P, P, I, P, I, I, I, I, I, F, I, I, P]
    lib.ns_attention_decode_noalloc.restype = c_int
    lib.ns_attention_decode.argtypes = [P, I, P, P, P, I, P, P, P, P, I, P, P, P, P, I, I, I, I, I, F, I, I, P]
    lib.ns_attention_decode.restype = c_int
    lib.ns_last_error.restype = ctypes.c_char_p
    return lib


def _problem(n_req, S, nq, nkv, d, page, seed):
    g = torch.Generator().manual_seed(seed)
    n_pages = n_req * (-(-S // page)) + 5
    kc = (torch.randn(n_pages, nkv, page, d, generator=g)).to(torch.bfloat16).to(DEV)  # [page, kv head, offset, dim]
    vc = (torch.randn(n_pages, nkv, page, d, generator=g)).to(torch.bfloat16).to(DEV)
    perm = torch.randperm(n_pages, generator=g)
    width = -(-S // page)
    tables = perm[: n_req * width].view(n_req, width).to(torch.int32).to(DEV)
    lens = [S - 7 * (r % 4) for r in range(n_req)]
    q = torch.randn(n_req, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16).to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return dict(q=q, kc=kc, vc=vc, tables=tables, token_req=i32(list(range(n_req))), positions=i32([n - 1 for n in lens]),
                qo=i32(list(range(n_req + 1))), n=n_req, nq=nq, nkv=nkv, d=d, page=page, lens=lens)


def _plain(p):
    """softmax(q k^T / sqrt(d)) v per request over the keys gathered from its pages, in float32."""
    import plain_llama as plain
    nq, nkv, d = p["nq"], p["nkv"], p["d"]
    out = []
    for r, n in enumerate(p["lens"]):
        pages = p["tables"][r].long()
        k = p["kc"][pages].permute(0, 2, 1, 3).reshape(-1, nkv, d)[:n].float()   # [keys, kv head, dim]
        v = p["vc"][pages].permute(0, 2, 1, 3).reshape(-1, nkv, d)[:n].float()
        q = torch.zeros(n, nq, d, device=DEV)
        q[-1] = p["q"][r, : nq * d].float().view(nq, d)                            # the one query sits at the last position
        out.append(plain.plain_attention(q, k, v)[-1].reshape(-1))
    return torch.stack(out)


def _run(lib, p, n_splits, no_alloc):
    out = torch.zeros(p["n"], p["nq"] * p["d"], dtype=torch.bfloat16, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    head = (p["q"].data_ptr(), p["q"].stride(0), p["kc"].data_ptr(), p["vc"].data_ptr(), p["tables"].data_ptr(),
            p["tables"].stride(0), p["token_req"].data_ptr(), p["positions"].data_ptr(), p["qo"].data_ptr(),
            out.data_ptr(), out.stride(0))
    tail = (None, p["n"], p["nq"], p["nkv"], p["d"], p["page"], 1.0 / math.sqrt(p["d"]), 0, n_splits, stream)
    if no_alloc:
        rc = lib.ns_attention_decode_noalloc(*head, *tail)
    else:
        rows = p["n"] * p["nq"] * n_splits
        part_o = torch.empty(rows, p["d"], dtype=torch.float32, device=DEV)
        part_ml = torch.empty(rows, 2, dtype=torch.float32, device=DEV)
        counters = torch.zeros(p["n"] * p["nkv"], dtype=torch.int32, device=DEV)
        rc = lib.ns_attention_decode(*head, part_o.data_ptr(), part_ml.data_ptr(), counters.data_ptr(), *tail)
    torch.cuda.synchronize()
    return rc, out


def test_no_alloc_entry_point_matches_the_allocating_one_on_two_calls_in_a_row():
    lib = _lib()
    first = _problem(n_req=5, S=900, nq=8, nkv=2, d=128, page=16, seed=1)
    second = _problem(n_req=3, S=333, nq=12, nkv=4, d=64, page=8, seed=2)  # other sizes on the same array
    for p, n_splits in ((first, 8), (second, 3), (first, 2)):
        rc, got = _run(lib, p, n_splits, no_alloc=True)
        assert rc == 0, lib.ns_last_error().decode()
        rc, want = _run(lib, p, n_splits, no_alloc=False)
        assert rc == 0, lib.ns_last_error().decode()
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=3e-2)
        assert torch.equal(got, want)  # same kernel, same order of sums: the same bits
        torch.testing.assert_close(got.float(), _plain(p), rtol=2e-2, atol=2e-2)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    p = _problem(n_req=64, S=40, nq=32, nkv=8, d=128, page=16, seed=3)
    need = 4 * 64 * 32 * 16 * (128 + 2)
    assert need > NO_ALLOC_BYTES
    rc, _ = _run(lib, p, 16, no_alloc=True)
    assert rc != 0
    msg = lib.ns_last_error().decode()
    assert "8388608" in msg and "scratch" in msg
    rc, got = _run(lib, p, 2, no_alloc=True)  # the same problem with fewer splits fits
    assert rc == 0, lib.ns_last_error().decode()
    rc, want = _run(lib, p, 2, no_alloc=False)
    assert torch.equal(got, want)
    torch.testing.assert_close(got.float(), _plain(p), rtol=2e-2, atol=2e-2)
    # one split shares nothing between blocks: no scratch, so no size is too large
    big = _problem(n_req=600, S=40, nq=32, nkv=8, d=128, page=16, seed=4)
    rc, got = _run(lib, big, 1, no_alloc=True)
    assert rc == 0, lib.ns_last_error().decode()
    torch.testing.assert_close(got.float(), _plain(big), rtol=2e-2, atol=2e-2)
    # and what the kernel refuses is refused before anything reaches the stream
    rc, _ = _run(lib, p, 17, no_alloc=True)
    assert rc != 0 and "n_splits" in lib.ns_last_error().decode()

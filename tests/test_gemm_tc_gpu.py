"""The tcgen05 matrix product alone against float64 arithmetic on the same bf16 inputs: few
tokens (weight streaming), many tokens (tiled), sizes that are no multiple of any tile, split-K over
a thread-block cluster, float32 output, and operands that TMA cannot take (refused, then
served by the fallback)."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ops():
    from nanospec_b200 import ops as o
    return o


def case(M, N, K, seed, ldx=None, ldw=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, ldx or K, generator=g).to(torch.bfloat16).to(DEV)[:, :K]
    w = torch.randn(N, ldw or K, generator=g).to(torch.bfloat16).to(DEV)[:, :K]
    return x, w, x.double() @ w.double().T


def check(out, want, K):
    err = (out.double() - want).abs().max().item()
    scale = want.abs().max().item()
    tol = (2.0 ** -8 if out.dtype == torch.bfloat16 else 1e-5) * scale + 1e-4 * K ** 0.5
    assert err <= tol, f"max |diff| {err} against tolerance {tol}"


def test_smallest_tile_first():
    x, w, want = case(8, 128, 64, 0)
    out = torch.zeros(8, 128, dtype=torch.float32, device=DEV)
    assert ops().linear_tensor_core(x, w, out, splits=1)
    torch.cuda.synchronize()
    ops().check_kernel_errors()
    check(out, want, 64)


@pytest.mark.parametrize("M,N,K", [
    (1, 256, 256), (8, 6144, 4096), (3, 331, 96), (16, 128, 4096), (17, 200, 520), (40, 1000, 1024), (64, 4096, 1024),
    (100, 384, 200), (130, 257, 72), (300, 512, 1024), (700, 1152, 2048), (2048, 1024, 512),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_against_float64(M, N, K, out_dtype):
    x, w, want = case(M, N, K, M + N + K)
    out = torch.full((M, N), 7.0, dtype=out_dtype, device=DEV)
    assert ops().linear_tensor_core(x, w, out, splits=1)
    torch.cuda.synchronize()
    ops().check_kernel_errors()
    check(out, want, K)


@pytest.mark.parametrize("M,N,K,splits", [(8, 4096, 4096, 4), (1, 512, 14336, 8), (64, 384, 1024, 2), (20, 200, 520, 2), (8, 256, 8192, 8),
                                          (33, 331, 1024, 4), (16, 6144, 4096, 2)])
def test_split_k_over_a_cluster_is_deterministic(M, N, K, splits):
    x, w, want = case(M, N, K, splits)
    outs = []
    for _ in range(3):
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        assert ops().linear_tensor_core(x, w, out, splits=splits)
        outs.append(out)
    torch.cuda.synchronize()
    ops().check_kernel_errors()
    check(outs[0], want, K)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("M,inter,K,splits", [(1, 64, 64, 1), (8, 14336, 4096, 1), (16, 384, 1024, 2), (5, 128, 8192, 8), (40, 192, 520, 4),
                                              (300, 256, 256, 1)])
def test_gated_epilogue(M, inter, K, splits):
    """The packed projection with gate and up rows alternating in runs of 64: the kernel's epilogue applies
    silu(gate) * up; against float64, and against the unfused product followed by the swiglu kernel."""
    g = torch.Generator().manual_seed(inter + M)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(inter, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16).to(DEV)
    up = (torch.randn(inter, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16).to(DEV)
    w = torch.stack([gate.view(inter // 64, 64, K), up.view(inter // 64, 64, K)], dim=1).reshape(2 * inter, K).contiguous()
    gd, ud = x.double() @ gate.double().T, x.double() @ up.double().T
    want = gd / (1 + torch.exp(-gd)) * ud
    o = ops()
    out = torch.full((M, inter), 7.0, dtype=torch.bfloat16, device=DEV)
    o.lib.call("ns_gemm_bf16_tc_gated", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, 2 * inter, K, x.stride(0), w.stride(0),
               out.stride(0), 0, splits, o._tc(torch.device(DEV)).error.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    o.check_kernel_errors()
    err = (out.double() - want).abs().max().item()
    assert err <= 2.0 ** -8 * want.abs().max().item() + 1e-3, err
    # the two-kernel path on the same packed weights (it rounds the products to bf16 first)
    scratch = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device=DEV)
    out2 = torch.empty_like(out)
    o.swiglu(o.linear(x, w, scratch), out2, 64)
    torch.testing.assert_close(out2.float(), want.float(), rtol=3e-2, atol=3e-2)
    # and what the part calls
    out3 = torch.empty_like(out)
    o.gated_linear(x, w, out3, scratch, 64)
    if M <= 16:
        assert torch.equal(out3, out) or splits != o.gemm_splits(M, 2 * inter, K)
    torch.testing.assert_close(out3.float(), want.float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("M,H,K,N2", [(1, 128, 64, 256), (8, 4096, 4096, 6144), (16, 256, 520, 384), (5, 384, 14336, 128),
                                      (30, 512, 1024, 256), (50, 256, 520, 384), (64, 4096, 4096, 6144)])
def test_norm_epilogues(M, H, K, N2, monkeypatch):
    """A product that feeds a norm sink (residual sum, gain, partial sums of squares) and the products
    that apply the missing per-row scale, plain and gated - against float64, twice for determinism."""
    from types import SimpleNamespace
    from nanospec_b200.parts import Workspace
    o = ops()
    g = torch.Generator().manual_seed(M + H)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(H, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    resid0 = torch.randn(M, H, generator=g).to(DEV)
    gain = (1 + 0.1 * torch.randn(H, generator=g)).to(DEV)
    w2 = (torch.randn(N2, H, generator=g) / H ** 0.5).to(torch.bfloat16).to(DEV)
    eps = 1e-5
    ws = Workspace(torch.device(DEV))
    monkeypatch.setattr(o, "TENSOR_CORE_GEMM_MAX_TOKENS", 64)  # the kernel's own limit, whatever the engine's choice of library is
    assert o.norm_fusion_ok(M, torch.bfloat16, w, w2)
    r_want = resid0.double() + x.double() @ w.double().T
    scale = torch.rsqrt((r_want ** 2).mean(dim=1, keepdim=True) + eps)
    results = []
    for _ in range(2):
        resid = resid0.clone()
        rs = o.linear(x, w, torch.empty(M, H, dtype=torch.bfloat16, device=DEV), sink=o.NormSink(resid, gain, eps, ws))
        assert isinstance(rs, o.RowScaled) and rs.gain is gain
        torch.testing.assert_close(resid.double(), r_want, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(rs.x.double(), (gain.double() * r_want), rtol=2 ** -7, atol=1e-3)
        got_scale = torch.rsqrt(rs.partials.double().sum(dim=1, keepdim=True) / H + eps)
        torch.testing.assert_close(got_scale, scale, rtol=1e-5, atol=0)
        out2 = o.linear(rs, w2, torch.empty(M, N2, dtype=torch.bfloat16, device=DEV))
        want2 = (rs.x.double() * scale) @ w2.double().T          # the kernel sees the rounded gain * resid
        check(out2, want2, H)
        results.append((resid.clone(), rs.x.clone(), rs.partials.clone(), out2.clone()))
        # gated, on the same activations: N2 packed features = N2 / 2 outputs
        outg = torch.empty(M, N2 // 2, dtype=torch.bfloat16, device=DEV)
        o.gated_linear(rs, w2, outg, torch.empty(M, N2, dtype=torch.bfloat16, device=DEV), 64)
        full = want2.view(M, N2 // 128, 2, 64)
        gd, ud = full[:, :, 0].reshape(M, -1), full[:, :, 1].reshape(M, -1)
        torch.testing.assert_close(outg.double(), gd / (1 + torch.exp(-gd)) * ud, rtol=2 ** -6, atol=2e-2)
    torch.cuda.synchronize()
    o.check_kernel_errors()
    for a, b in zip(*results):
        assert torch.equal(a, b)


@pytest.mark.parametrize("M,nq,nkv,d,K,page", [(1, 4, 2, 64, 256, 8), (8, 32, 8, 128, 4096, 16), (20, 8, 4, 32, 520, 4), (33, 2, 1, 128, 128, 16),
                                                  (40, 8, 4, 64, 520, 8), (64, 32, 8, 128, 4096, 16)])
def test_rope_epilogue(M, nq, nkv, d, K, page):
    """The packed projection with rotation and cache write in its epilogue against the projection followed by
    the rotation kernel: the same q, the same pages (a padding row among the tokens is skipped)."""
    o = ops()
    g = torch.Generator().manual_seed(M + d)
    N = (nq + 2 * nkv) * d
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16).to(DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))).to(DEV)
    n_pages = M * 3 + 4
    positions = torch.randint(0, 3 * page, (M,), generator=g).to(torch.int32)
    token_req = torch.arange(M, dtype=torch.int32)
    if M > 4:
        token_req[3] = -1
    tables = torch.randperm(n_pages, generator=g)[: M * 3].to(torch.int32).view(M, 3).to(DEV)
    positions, token_req = positions.to(DEV), token_req.to(DEV)
    caches = []
    outs = []
    keep = o.TENSOR_CORE_GEMM_MAX_TOKENS
    o.TENSOR_CORE_GEMM_MAX_TOKENS = 64  # the kernel's own limit, whatever the engine's choice of library is
    try:
        for fused in (True, False):
            kc = torch.zeros(n_pages, nkv, page, d, dtype=torch.bfloat16, device=DEV)
            vc = torch.zeros_like(kc)
            out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
            if fused:
                assert o.linear_rope(x, w, out, positions, token_req, tables, inv_freq, kc, vc, page, nq, nkv, d)
            else:
                o.linear(x, w, out)
                o.rope_kv_write(out, positions, token_req, tables, inv_freq, kc, vc, page, nq, nkv, d)
            torch.cuda.synchronize()
            o.check_kernel_errors()
            outs.append(out[:, : nq * d].float())
            caches.append((kc.float(), vc.float()))
    finally:
        o.TENSOR_CORE_GEMM_MAX_TOKENS = keep
    live = (token_req >= 0)
    # the fused epilogue rotates the fp32 sums; the two-kernel path rounds them to bf16 first
    torch.testing.assert_close(outs[0][live], outs[1][live], rtol=2 ** -6, atol=2e-2)
    torch.testing.assert_close(caches[0][0], caches[1][0], rtol=2 ** -6, atol=2e-2)
    torch.testing.assert_close(caches[0][1], caches[1][1], rtol=2 ** -6, atol=2e-2)
    assert float(caches[0][0].abs().sum()) > 0
    # and against float64 for the keys: rotate the exact products
    full = x.double() @ w.double().T
    k = full[:, nq * d: (nq + nkv) * d].view(M, nkv, d)
    ang = positions.double()[:, None] * inv_freq.double()[None, :]
    c, s_ = ang.cos()[:, None, :], ang.sin()[:, None, :]
    k_rot = torch.cat([k[..., : d // 2] * c - k[..., d // 2:] * s_, k[..., d // 2:] * c + k[..., : d // 2] * s_], dim=-1)
    for n in range(M):
        if int(token_req[n]) < 0:
            continue
        pg = int(tables[n, int(positions[n]) // page])
        got = caches[0][0][pg, :, int(positions[n]) % page, :]
        torch.testing.assert_close(got.double(), k_rot[n], rtol=2 ** -7, atol=1e-2)


def test_strided_rows_and_output():
    x, w, want = case(24, 192, 128, 5, ldx=136, ldw=256)
    wide = torch.zeros(24, 400, dtype=torch.bfloat16, device=DEV)
    out = wide[:, 100:292]
    assert ops().linear_tensor_core(x, w, out, splits=1)
    torch.cuda.synchronize()
    check(out, want, 128)
    assert float(wide[:, :100].abs().max()) == 0 and float(wide[:, 292:].abs().max()) == 0


def test_operands_tma_cannot_take_fall_back():
    x, w, want = case(5, 64, 100, 9)  # K = 100 is no multiple of 8
    out = torch.zeros(5, 64, dtype=torch.bfloat16, device=DEV)
    assert not ops().linear_tensor_core(x, w, out)
    ops().linear(x.contiguous(), w.contiguous(), out)
    check(out, want, 100)
    assert ops().gemm_splits(8, 4096, 4096) > 1 and ops().gemm_splits(2048, 4096, 4096) == 1

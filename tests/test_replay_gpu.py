"""Trace replay on the GPU against the plain implementation: the same sequences whole, with
the last 32 tokens one by one, in portions of changing size, and mixed with other requests
on a pool so small that pages are used again - in float32 and in bfloat16, for three tiny
configurations."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_llama as plain
from conftest import TINY, random_ids
from trace_util import collect, peak_tokens, run_trace, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu

# float32: both sides are true fp32; only the order of sums differs.
F32_TOL = 2e-5
# bfloat16: the reference's own bound for its kernels against an fp32-exact oracle is 8 bf16
# ulps of the row's largest logit (tests/conftest.py:25-26,58-77 there), median <= 2.
BF16_ULP = 2.0 ** -7


def sequences(name: str) -> tuple[dict[str, list[int]], dict[str, int]]:
    cfg = TINY[name]["config"]
    lens = {"A": [5, 17, 33, 64 + 16, 130], "B": [1, 9, 40, 100, 130, 250], "C": [3, 50, 77, 200, 36]}[name]
    seqs, prompts = {}, {}
    for i, n in enumerate(lens):
        total = min(n + 34, cfg.max_position_embeddings)
        seqs[f"r{i}"] = random_ids(total, cfg.vocab_size, seed=1000 + 17 * i + TINY[name]["seed"])
        prompts[f"r{i}"] = min(n, total)
    return seqs, prompts


_plain_cache: dict[str, dict[str, np.ndarray]] = {}


def plain_logits(name: str, folder) -> dict[str, np.ndarray]:
    if name not in _plain_cache:
        cfg, w = plain.read_folder(folder)
        seqs, _ = sequences(name)
        _plain_cache[name] = {r: plain.plain_forward(cfg, w, ids).numpy() for r, ids in seqs.items()}
    return _plain_cache[name]


def check(got: dict[str, np.ndarray], want: dict[str, np.ndarray], dtype: str, what: str) -> None:
    for r in want:
        g, w = got[r], want[r]
        assert g.shape == w.shape
        rowmax = np.abs(w).max(axis=1, keepdims=True)
        err = np.abs(g - w)
        if dtype == "float32":
            bad = err > F32_TOL * np.maximum(rowmax, 1.0)
            assert not bad.any(), (f"{what}: request {r}: first wrong position {int(np.argwhere(bad.any(axis=1))[0][0])}, "
                                   f"max |diff| {err.max():.3g}")
        else:
            ulps = err / (BF16_ULP * rowmax)
            worst = ulps.max(axis=1)
            assert worst.max() <= 8.0, (f"{what}: request {r}: position {int(worst.argmax())} is {worst.max():.2f} "
                                        f"bf16 ulps of the row maximum away")
            assert np.median(worst) <= 2.0, f"{what}: request {r}: median of the worst ulps per row {np.median(worst):.2f}"


CUTS = {
    "whole": lambda seqs, prompts: trace_whole(seqs),
    "tail32": lambda seqs, prompts: trace_tail(seqs, 32),
    "portions": lambda seqs, prompts: trace_portions(seqs),
    "mixed": lambda seqs, prompts: trace_mixed(seqs, prompts, max_live=4),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_every_cut(name, dtype, tiny_folders, tmp_path):
    folder = tiny_folders[name]
    seqs, prompts = sequences(name)
    want = plain_logits(name, folder)
    page = TINY[name]["page"]
    for cut, make in CUTS.items():
        steps = make(seqs, prompts)
        # the pool holds exactly the peak of the trace, so finished requests' pages are used again
        budget = peak_tokens(steps)
        results = run_trace(folder, dtype, steps, budget, tmp_path / f"{cut}", block_size=page,
                            vocab=TINY[name]["config"].vocab_size)
        check(collect(steps, results, seqs), want, dtype, f"config {name} {dtype} {cut}")


def test_cuts_agree_bit_for_bit_in_float32(tiny_folders, tmp_path):
    """In float32 every sum runs in an order that does not depend on the cut, so the cuts
    must agree far below the tolerance against the plain implementation."""
    name = "B"
    folder = tiny_folders[name]
    seqs, prompts = sequences(name)
    page = TINY[name]["page"]
    outs = {}
    for cut in ("whole", "mixed"):
        steps = CUTS[cut](seqs, prompts)
        res = run_trace(folder, "float32", steps, peak_tokens(steps), tmp_path / cut, block_size=page)
        outs[cut] = collect(steps, res, seqs)
    for r in seqs:
        assert np.array_equal(outs["whole"][r], outs["mixed"][r]), f"request {r} differs between cuts"

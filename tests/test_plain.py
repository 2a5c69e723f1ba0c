"""The plain implementation against its recorded outputs (tests/golden/plain_outputs.json,
made by tests/golden/make_golden.py after comparing with the reference's own code), against
the reference itself when its tree is present, and against hand-checkable cases (no GPU)."""

from __future__ import annotations

import json
import math
import os
import sys
from pathlib import Path

import pytest
import torch

import plain_llama as plain
from conftest import TINY

GOLDEN = json.loads((Path(__file__).parent / "golden" / "plain_outputs.json").read_text())


@pytest.mark.parametrize("name", list(TINY))
def test_plain_matches_recorded_outputs(name, tiny_folders):
    rec = GOLDEN[name]
    assert rec["seed"] == TINY[name]["seed"] and rec["max_abs_diff_to_reference"] < 2e-5
    cfg, w = plain.read_folder(tiny_folders[name])
    logits = plain.plain_forward(cfg, w, rec["prompt"])
    got = [float(logits[-1, i]) for i in rec["probe_vocab_entries"]]
    assert max(abs(a - b) for a, b in zip(got, rec["last_logits_at_probe"])) < 2e-6
    greedy, _ = plain.plain_greedy(cfg, w, rec["prompt"], len(rec["greedy_8"]))
    assert greedy == rec["greedy_8"]
    for d in rec["draws"]:
        lp = plain.plain_process(logits[-1], d["temperature"], d["top_k"], d["top_p"])
        assert plain.plain_draw(lp, d["u"]) == d["token"]


def test_inverse_frequencies_bands():
    inv = plain.plain_inv_freq(32, 500000.0, {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                              "original_max_position_embeddings": 64})
    base = plain.plain_inv_freq(32, 500000.0, None)
    wavelen = 2 * math.pi / base
    assert torch.equal(inv[wavelen < 16], base[wavelen < 16])                 # short waves untouched
    assert torch.allclose(inv[wavelen > 64], base[wavelen > 64] / 8.0)         # long waves divided by the factor
    mid = (wavelen >= 16) & (wavelen <= 64)
    assert mid.any() and ((inv[mid] <= base[mid]) & (inv[mid] >= base[mid] / 8.0)).all()


def test_attention_causal_window_and_groups():
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(6, 4, 8, generator=g), torch.randn(6, 2, 8, generator=g), torch.randn(6, 2, 8, generator=g)
    out = plain.plain_attention(q, k, v)
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0), atol=1e-6)  # the first query sees only key 0
    w1 = plain.plain_attention(q, k, v, window=1)
    assert torch.allclose(w1, v.repeat_interleave(2, dim=1), atol=1e-6)         # window 1: each query sees itself
    # heads 0,1 read kv head 0 and heads 2,3 read kv head 1
    k2 = k.clone()
    k2[:, 1] *= 3.0
    out2 = plain.plain_attention(q, k2, v)
    assert torch.allclose(out2[:, :2], out[:, :2], atol=1e-6) and not torch.allclose(out2[:, 2:], out[:, 2:])


def test_process_by_hand():
    z = torch.tensor([2.0, 1.0, 0.0, -1.0])
    lp = plain.plain_process(z, 0.5)
    assert torch.allclose(lp, torch.log_softmax(z / 0.5, -1))
    lp = plain.plain_process(z, 1.0, top_k=2)
    assert torch.isinf(lp[2:]).all() and torch.allclose(lp[:2].exp().sum(), torch.tensor(1.0))
    p = torch.softmax(z, -1)  # 0.644, 0.237, 0.087, 0.032
    lp = plain.plain_process(z, 1.0, top_p=0.7)  # token 1 starts below 0.7, token 2 starts at 0.88
    assert torch.isfinite(lp[:2]).all() and torch.isinf(lp[2:]).all()
    assert plain.plain_draw(torch.log(p), 0.0) == 0 and plain.plain_draw(torch.log(p), 0.65) == 1
    assert plain.plain_draw(torch.log(p), 0.9999999) == 3


# the reference's source tree: $NANOSPEC_REFERENCE, or a folder `reference` beside this repository
REFERENCE = Path(os.environ.get("NANOSPEC_REFERENCE", Path(__file__).resolve().parents[2] / "reference"))


@pytest.mark.skipif(not (REFERENCE / "model" / "llama.py").is_file(), reason="the reference tree is not here")
def test_plain_matches_the_reference_code(tiny_folders):
    sys.path.insert(0, str(REFERENCE))
    try:
        from kv.allocator import BlockAllocator
        from kv.cache import AttnMeta, PagedKVCache
        from model.loader import load_model
    finally:
        sys.path.remove(str(REFERENCE))
    ref = load_model(tiny_folders["B"], device="cpu", dtype=torch.float32, backend="sdpa")
    cfg, w = plain.read_folder(tiny_folders["B"])
    ids = GOLDEN["B"]["prompt"]
    alloc, kv = BlockAllocator(32, 8), PagedKVCache(ref.config, 32, 8, "cpu", torch.float32)
    meta = AttnMeta.build([alloc.alloc(0, len(ids))], [len(ids)], 8, "cpu")
    want, _ = ref(torch.tensor(ids), kv, meta)
    assert (plain.plain_forward(cfg, w, ids) - want).abs().max() < 2e-5

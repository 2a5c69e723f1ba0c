"""The layer widths of the benchmark configuration (hidden 4096, 32 query heads over 8 kv heads of 128, an
intermediate size of 14336, llama3-scaled rotary frequencies, pages of 16) with two layers, a vocabulary that
is no power of two and seeded random weights: trace replay against the plain implementation in float32 and in
bfloat16, whole, with a decoded tail, and mixed on a small pool.  The tiny configurations never reach the
kernels that these sizes select (TMA decode attention in a cluster, tcgen05 prefill attention, the products'
gated, norm and rotation epilogues); this does."""

from __future__ import annotations

import numpy as np
import pytest

import plain_llama as plain
from conftest import random_ids
from test_replay_gpu import check
from trace_util import collect, peak_tokens, run_trace, trace_mixed, trace_tail, trace_whole

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from nanospec_b200.config import Llama3RopeScaling, LlamaConfig
    from nanospec_b200.weights import write_random_model
    cfg = LlamaConfig(vocab_size=20011, hidden_size=4096, intermediate_size=14336, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=1024, rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 256),
                      tie_word_embeddings=True)
    d = tmp_path_factory.mktemp("flagship_widths")
    write_random_model(d, cfg, seed=21)
    return d


@pytest.fixture(scope="module")
def case(folder):
    lens = {"long": 300, "mid": 75, "short": 9}
    seqs = {name: random_ids(n + 20, 20011, seed=500 + n) for name, n in lens.items()}
    cfg, w = plain.read_folder(folder)
    want = {r: plain.plain_forward(cfg, w, ids).numpy() for r, ids in seqs.items()}
    return seqs, lens, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_at_the_benchmark_widths(dtype, folder, case, tmp_path):
    seqs, prompts, want = case
    cuts = {
        "whole": trace_whole(seqs),
        "tail": trace_tail(seqs, 20),
        "mixed": trace_mixed(seqs, prompts, max_live=3, portions=(64, 2, 130, 17)),
    }
    for cut, steps in cuts.items():
        results = run_trace(folder, dtype, steps, peak_tokens(steps), tmp_path / cut, block_size=16, vocab=20011)
        check(collect(steps, results, seqs), want, dtype, f"benchmark widths {dtype} {cut}")

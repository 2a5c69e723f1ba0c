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
def folder(wide_folders):
    return wide_folders["wide128"]


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


def test_the_whole_benchmark_shape_in_float32_under_every_cut():
    """All 32 layers of the benchmark shape in true float32 (32 GB of random weights drawn on the device), short
    requests, the four ways of cutting the work.  Sums of 14,336 terms through 32 layers move float32 results by
    more than the tiny models' bound, whatever the order of summation, so the yardstick here is float64: the plain
    implementation runs on the same GPU with the very tensors the engine holds, once in float64 (the truth) and
    once in float32 (a library's order of summation), and the engine must be as close to the truth as that is,
    within a factor of three.  And the cuts must agree with each other bit for bit."""
    import torch

    from nanospec_b200.config import Llama3RopeScaling, LlamaConfig
    from nanospec_b200.engine import ModelRunner, StepEntry
    from nanospec_b200.weights import random_model
    from trace_util import trace_portions

    if torch.cuda.mem_get_info()[0] < 100e9:
        pytest.skip("needs about 90 GB of free device memory")
    torch.backends.cuda.matmul.allow_tf32 = False
    cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=8192, rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 8192))
    model, w = random_model(cfg, seed=3, device="cuda", dtype=torch.float32, return_tensors=True)
    pcfg = {"layers": 32, "heads": 32, "kv_heads": 8, "head_dim": 128, "eps": 1e-5, "theta": 500000.0,
            "scaling": {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}}

    class AsDouble(dict):  # the same tensors, converted as they are used
        def __getitem__(self, k):
            return dict.__getitem__(self, k).double()

    lens = {"a": 60, "b": 33, "c": 5}
    seqs = {name: random_ids(n + 6, 128256, seed=900 + n) for name, n in lens.items()}
    truth = {r: plain.plain_forward(pcfg, AsDouble(w), ids).cpu().numpy() for r, ids in seqs.items()}
    plain32 = {r: plain.plain_forward(pcfg, w, ids).cpu().numpy().astype(np.float64) for r, ids in seqs.items()}
    cuts = {
        "whole": trace_whole(seqs),
        "tail": trace_tail(seqs, 6),
        "portions": trace_portions(seqs),
        "mixed": trace_mixed(seqs, lens, max_live=3, portions=(13, 2, 32, 6)),
    }
    got = {}
    for cut, steps in cuts.items():
        runner = ModelRunner(model, num_blocks=max(1, -(-peak_tokens(steps) // 16)), block_size=16, max_requests=4)
        ids, results = {}, {}
        for rec in steps:
            entries = []
            for e in rec["entries"]:
                if e["id"] not in ids:
                    ids[e["id"]] = len(ids)
                    runner.begin(ids[e["id"]])
                entries.append(StepEntry(ids[e["id"]], e["tokens"], e.get("want", [])))
            out = runner.step(entries)
            if out is not None:
                results[rec["step"]] = out.float().cpu().numpy()
            for name in rec["end"]:
                runner.end(ids[name])
        runner.manager.check()
        got[cut] = collect(steps, results, seqs)
    for r in seqs:
        yard = np.abs(plain32[r] - truth[r]).max()
        print(f"request {r}: plain float32 is {yard:.3g} from float64, the engine "
              f"{np.abs(got['whole'][r].astype(np.float64) - truth[r]).max():.3g} (largest logit {np.abs(truth[r]).max():.3g})")
        for cut in cuts:
            err = np.abs(got[cut][r].astype(np.float64) - truth[r]).max()
            assert err <= 3.0 * yard, f"{cut}: request {r}: {err:.3g} from float64, plain float32 is {yard:.3g} from it"
            assert np.array_equal(got[cut][r], got["whole"][r]), f"request {r}: cut {cut} differs from the whole prompt"
    del model, w, runner
    torch.cuda.empty_cache()  # tests after this one start their own processes on the same GPU

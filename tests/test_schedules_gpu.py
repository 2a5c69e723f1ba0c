"""Schedules and sizes that the other GPU tests do not reach, each against the plain implementation:
generation at real layer widths through CUDA graphs and steps launched ahead, graphs captured at first use
while the batch grows, heads of 64 as a whole model, a hundred requests decoding in one eager step beside
portions of prompts, positions in the thousands, the head in chunks, the phase timers, pages that are handed
out again, and the command line on the GPU.  In the manner of the reference's tests/test_correctness.py:25-80,
tests/test_batching.py:29-74 and tests/test_graphs.py:34-72, on seeded random models."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as plain
from conftest import ROOT, TINY, WIDE, random_ids
from test_replay_gpu import BF16_ULP, F32_TOL, check
from trace_util import collect, peak_tokens, replay_in_process, run_trace, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def load(folder, dtype):
    from nanospec_b200 import load_model
    return load_model(folder, device="cuda", dtype=dtype)


def engine(model, **kw):
    from nanospec_b200 import Engine, EngineConfig
    return Engine(model, EngineConfig(**kw))


def params(**kw):
    from nanospec_b200 import SamplingParams
    return SamplingParams(**kw)


def plain_on_gpu(folder):
    cfg, w = plain.read_folder(folder)
    torch.backends.cuda.matmul.allow_tf32 = False
    return cfg, {k: v.cuda() for k, v in w.items()}


def check_rows(got: np.ndarray, want: np.ndarray, dtype: torch.dtype, what: str) -> None:
    """Rows of logits against the plain implementation's, by the rule of the replay tests."""
    check({"x": got}, {"x": want}, "float32" if dtype == torch.float32 else "bfloat16", what)


def check_teacher_forced(reqs, prompts, cfg, w, dtype, what: str) -> None:
    """Every step's recorded logits of every request against the plain implementation run over the request's
    own tokens (prompt + what the engine emitted): a token that differs from the plain argmax at a near-tie
    does not make the rest of the sequence incomparable."""
    for i, (req, prompt) in enumerate(zip(reqs, prompts)):
        ids = list(prompt) + req.out_tokens
        want = plain.plain_forward(cfg, w, ids[:-1])[len(prompt) - 1:].cpu().numpy()
        got = torch.stack(req.step_logits).numpy()
        assert got.shape == want.shape, (what, i, got.shape, want.shape)
        check_rows(got, want, dtype, f"{what}: request {i}")
        # and the emitted token is the argmax of the engine's own logits
        assert req.out_tokens == got.argmax(axis=1).tolist(), f"{what}: request {i}"


# ---------------------------------------------------------------------------------------------------
# graphs and steps launched ahead at the widths that select the fused kernels
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_at_benchmark_widths_through_graphs_and_lookahead(dtype, wide_folders):
    """Five requests of different lengths and limits, so that the live count falls 5 -> 4 -> 3 -> 2 -> 1 (buckets 8,
    4, 4, 2, 1 with padding rows) over 50 decode steps.  What bench.py times - `Engine.step` with graph replay,
    padding rows, token ids taken on the device, steps launched ahead - gives the same tokens with and without
    launching ahead, and every step's logits lie within the kernels' bound of the plain implementation's."""
    dt = DTYPES[dtype]
    folder = wide_folders["wide128"]
    cfg, w = plain_on_gpu(folder)
    model = load(folder, dt)
    vocab = WIDE["wide128"].vocab_size
    prompts = [random_ids(n, vocab, seed=300 + n) for n in (5, 40, 130, 260, 17)]
    limits = [50, 6, 12, 24, 3]
    plist = [params(max_tokens=n) for n in limits]
    combos = [(True, True), (True, False), (False, True), (False, False)] if dtype == "bfloat16" else [(True, True), (False, False)]
    tokens = {}
    for graphs, ahead in combos:
        eng = engine(model, num_blocks=64, block_size=16, cuda_graphs=graphs, lookahead=ahead, max_admit=8)
        tokens[(graphs, ahead)] = eng.generate(prompts, plist)
        assert [len(t) for t in tokens[(graphs, ahead)]] == limits
        if ahead:
            assert eng.launched_ahead >= 30
        if graphs:
            assert {8, 4, 2, 1} <= set(eng.graphs.buckets) and eng.graphs.replays >= 45
        eng.cache.check()
        assert eng.cache.live == []
    # launching ahead replays the same kernels on the same inputs
    if dtype == "bfloat16":
        assert tokens[(True, True)] == tokens[(True, False)] and tokens[(False, True)] == tokens[(False, False)]
    # per-step logits, with and without graphs (recording them keeps the engine from launching ahead)
    for graphs in (True, False):
        eng = engine(model, num_blocks=64, block_size=16, cuda_graphs=graphs, record_logits=True, max_admit=8)
        reqs = [eng.add(p, s) for p, s in zip(prompts, plist)]
        while eng.sched.has_work:
            eng.step()
        assert [r.out_tokens for r in reqs] == tokens[(graphs, graphs)]
        check_teacher_forced(reqs, prompts, cfg, w, dt, f"wide128 {dtype} graphs={graphs}")


def test_graphs_captured_at_first_use_while_the_batch_grows(tmp_path):
    """`capture_at_start=False`: the bucket of 4 is captured first, then those of 32 and of 64 as the live count
    climbs 3 -> 20 -> 40, and then the first graph is replayed again when it has fallen back to 3.  Every bucket
    has scratch of its own that nothing can move once the graph points into it."""
    from nanospec_b200.config import LlamaConfig
    from nanospec_b200.weights import write_random_model

    cfg_t = LlamaConfig(vocab_size=1000, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=256)
    write_random_model(tmp_path, cfg_t, seed=5)
    cfg, w = plain_on_gpu(tmp_path)
    model = load(tmp_path, torch.bfloat16)
    waves = [(3, 44), (17, 14), (20, 6)]  # (requests, new tokens each): 3 live, then 20, then 40, then 20, then 3

    def run(**kw):
        eng = engine(model, num_blocks=400, block_size=16, record_logits=True, max_admit=64, **kw)
        reqs, prompts, sizes = [], [], []
        for wave, (n, new) in enumerate(waves):
            for i in range(n):
                prompts.append(random_ids(4 + (7 * i + wave) % 23, 1000, seed=1000 * wave + i))
                reqs.append(eng.add(prompts[-1], params(max_tokens=new)))
            for _ in range(6):
                eng.step()
                sizes.append(len(eng.sched.running))
        while eng.sched.has_work:
            eng.step()
            sizes.append(len(eng.sched.running))
        return eng, reqs, prompts, sizes

    eng, reqs, prompts, sizes = run(cuda_graphs=True, capture_at_start=False)
    assert max(sizes) == 40 and sizes[-2] == 3 and 20 in sizes
    assert list(eng.graphs.buckets) == [4, 32, 64], "buckets in the order of their first use"
    assert all(b.workspace.frozen for b in eng.graphs.buckets.values())
    assert len({id(b.workspace) for b in eng.graphs.buckets.values()} | {id(eng.runner.workspace)}) == 4
    check_teacher_forced(reqs, prompts, cfg, w, torch.bfloat16, "graphs at first use")
    _, eager_reqs, _, _ = run(cuda_graphs=False)
    check_teacher_forced(eager_reqs, prompts, cfg, w, torch.bfloat16, "eager")
    same = sum(a.out_tokens == b.out_tokens for a, b in zip(reqs, eager_reqs))
    assert same >= len(reqs) - 4  # a near-tie may fall differently: the graphs' attention splits the keys otherwise


@pytest.mark.parametrize("dtype,n_req", [("float32", 100), ("bfloat16", 100), ("bfloat16", 150)])
def test_more_than_64_requests_decode_from_the_larger_graphs(dtype, n_req, wide_folders):
    """The reference's graphs stop at 64 requests (engine/graphs.py:22); here 65 to 128 live requests replay the
    bucket of 128 and 129 to 256 that of 256, with their padding rows.  Every step's logits against the plain
    implementation."""
    dt = DTYPES[dtype]
    folder = wide_folders["wide64"]
    cfg, w = plain_on_gpu(folder)
    model = load(folder, dt)
    vocab = WIDE["wide64"].vocab_size
    prompts = [random_ids(3 + (11 * i) % 40, vocab, seed=7000 + i) for i in range(n_req)]
    plist = [params(max_tokens=3 + (i % 3) * 3) for i in range(n_req)]  # a third of them ends after 3 tokens, a third after 6
    top = 128 if n_req <= 128 else 256
    eng = engine(model, num_blocks=800, block_size=16, record_logits=True, max_admit=256, max_running=top)
    assert top in eng.graphs.buckets and 2 * top not in eng.graphs.buckets, "captured when the engine is built, up to max_running"
    reqs = [eng.add(p, s) for p, s in zip(prompts, plist)]
    sizes = []
    while eng.sched.has_work:
        eng.step()
        sizes.append(len(eng.sched.running))
    assert max(sizes) == n_req and eng.graphs.replays >= 7
    check_teacher_forced(reqs, prompts, cfg, w, dt, f"bucket of {top} {dtype}")
    eng.cache.check()
    assert eng.cache.live == []


def test_decode_rows_run_longest_context_first(tiny_folders):
    """A decode step's rows are ordered by context length, longest first (the order in which the decode attention
    kernel's blocks are scheduled), in graph replays and in eager steps alike; the tokens do not depend on it."""
    folder = tiny_folders["B"]
    spec = TINY["B"]
    cfg, w = plain.read_folder(folder)
    model = load(folder, torch.float32)
    vocab = spec["config"].vocab_size
    prompts = [random_ids(n, vocab, seed=40 + n) for n in (3, 30, 11, 30, 7)]
    for graphs in (True, False):
        eng = engine(model, num_blocks=64, block_size=spec["page"], cuda_graphs=graphs, max_admit=8)
        reqs = [eng.add(p, params(max_tokens=6)) for p in prompts]
        seen = 0
        while eng.sched.has_work:
            eng.step()
            flight = eng._inflight
            if flight is not None and all(len(s.tokens) == 1 for s in flight.batch):
                lengths = [s.req.committed for s in flight.batch]
                assert lengths == sorted(lengths, reverse=True), lengths
                seen += 1
        assert seen >= 3
        for req, p in zip(reqs, prompts):
            assert req.out_tokens == plain.plain_greedy(cfg, w, p, 6)[0]


@pytest.mark.parametrize("name", ["wide128", "wide64"])
def test_a_long_request_beside_short_ones_decodes_in_parts(name, tmp_path):
    """One context of 2,100 tokens among contexts of a few dozen: the packer cuts the long one into four parts, each an
    item of the decode attention kernel's work list, and the kernel adds the parts up.  Graph replays take the bucket's
    second graph (captured when it is first needed, in the middle of the run); eager steps take the list as it is.
    Every step's logits against the plain implementation; when the long request has ended the usual graph is back."""
    import dataclasses

    from nanospec_b200.weights import write_random_model

    write_random_model(tmp_path, dataclasses.replace(WIDE[name], max_position_embeddings=2304), seed=77)
    cfg, w = plain_on_gpu(tmp_path)
    model = load(tmp_path, torch.bfloat16)
    vocab = WIDE[name].vocab_size
    prompts = [random_ids(n, vocab, seed=500 + n) for n in (21, 2100, 33, 48, 5)]
    limits = [30, 12, 30, 30, 30]
    for graphs in (True, False):
        eng = engine(model, num_blocks=200, block_size=16, cuda_graphs=graphs, record_logits=True, max_admit=8)
        reqs = [eng.add(p, params(max_tokens=n)) for p, n in zip(prompts, limits)]
        while eng.sched.has_work:
            eng.step()
        if graphs:
            assert eng.graphs.buckets[8].graph_parts is not None and eng.graphs.buckets[4].graph_parts is None
            assert eng.graphs.replays >= 25
        check_teacher_forced(reqs, prompts, cfg, w, torch.bfloat16, f"{name}, a long request in parts, graphs={graphs}")
        eng.cache.check()
    # launched ahead, without the recorded logits: the same tokens (but for a near-tie)
    eng = engine(model, num_blocks=200, block_size=16, max_admit=8)
    outs = eng.generate(prompts, [params(max_tokens=n) for n in limits])
    assert sum(a == r.out_tokens for a, r in zip(outs, reqs)) >= 4
    assert eng.launched_ahead >= 20


def test_a_frozen_workspace_refuses_to_grow():
    from nanospec_b200.parts.context import Workspace

    ws = Workspace(torch.device("cuda"))
    a = ws.get("x", 4, 8, torch.float32)
    ws.frozen = True
    assert ws.get("x", 16, 8, torch.float32).data_ptr() == a.data_ptr()  # within what is there
    with pytest.raises(RuntimeError, match="would have to grow"):
        ws.get("x", 17, 8, torch.float32)


# ---------------------------------------------------------------------------------------------------
# heads of 64 as a whole model
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_heads_of_64(dtype, wide_folders, tmp_path):
    folder = wide_folders["wide64"]
    vocab = WIDE["wide64"].vocab_size
    lens = {"long": 280, "mid": 70, "short": 6, "late": 33}
    seqs = {name: random_ids(n + 34, vocab, seed=700 + n) for name, n in lens.items()}
    cfg, w = plain_on_gpu(folder)
    want = {r: plain.plain_forward(cfg, w, ids).cpu().numpy() for r, ids in seqs.items()}
    cuts = {
        "whole": trace_whole(seqs),
        "tail32": trace_tail(seqs, 32),
        "portions": trace_portions(seqs),
        "mixed": trace_mixed(seqs, lens, max_live=3, portions=(64, 2, 130, 17)),
    }
    for cut, steps in cuts.items():
        results = run_trace(folder, dtype, steps, peak_tokens(steps), tmp_path / cut, block_size=16, vocab=vocab)
        check(collect(steps, results, seqs), want, dtype, f"heads of 64, {dtype}, {cut}")
    if dtype == "bfloat16":
        # Portions this short make fewer blocks than the GPU has SMs and take the prefill kernel with one query head to
        # a block; once more with two heads to a block (what long prompts take), in this process
        from nanospec_b200 import ops
        model = load(folder, torch.bfloat16)
        ops.PREFILL_TWO_HEADS = "always"
        try:
            for cut in ("whole", "mixed"):
                steps = cuts[cut]
                results, _, _ = replay_in_process(model, steps, -(-peak_tokens(steps) // 16), 16)
                check(collect(steps, results, seqs), want, dtype, f"heads of 64, two heads to a block, {cut}")
        finally:
            ops.PREFILL_TWO_HEADS = "auto"


# ---------------------------------------------------------------------------------------------------
# more requests in one step than the largest graph holds
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_hundred_requests_decode_in_one_step_beside_two_portions(dtype, wide_folders):
    """100 requests with 3 to 42 tokens behind them bring one token each, a long prompt brings its second portion
    and a new request its first: one eager step, every logit against the plain implementation."""
    from nanospec_b200.engine import ModelRunner, StepEntry

    dt = DTYPES[dtype]
    folder = wide_folders["wide64"]
    vocab = WIDE["wide64"].vocab_size
    cfg, w = plain_on_gpu(folder)
    model = load(folder, dt)
    runner = ModelRunner(model, num_blocks=700, block_size=16, max_requests=102)
    seqs = {r: random_ids(4 + (r * 7) % 40, vocab, seed=2000 + r) for r in range(100)}
    seqs[100] = random_ids(228, vocab, seed=2100)
    seqs[101] = random_ids(77, vocab, seed=2101)
    for r in seqs:
        runner.begin(r)
    for lo in range(0, 100, 25):  # what came before, without logits
        assert runner.step([StepEntry(r, seqs[r][:-1]) for r in range(lo, lo + 25)]) is None
    assert runner.step([StepEntry(100, seqs[100][:100])]) is None
    entries = [StepEntry(r, seqs[r][-1:], [0]) for r in range(100)]
    entries.insert(37, StepEntry(100, seqs[100][100:], list(range(128))))
    entries.append(StepEntry(101, seqs[101], list(range(77))))
    out = runner.step(entries).float().cpu().numpy()
    assert out.shape == (100 + 128 + 77, vocab)
    row = 0
    for e in entries:
        n = len(e.want)
        want = plain.plain_forward(cfg, w, seqs[e.req_id]).cpu().numpy()[-n:]
        check_rows(out[row: row + n], want, dt, f"{dtype}: request {e.req_id} among 102 in one step")
        row += n
    for r in seqs:
        runner.end(r)
    runner.manager.check()
    if dtype != "bfloat16":
        return
    # The same steps again and again give the same bits.  Kernels overlap their predecessors' tails, so what runs
    # beside what changes from run to run; a wait inside a kernel that only holds for the usual timing shows up here
    # (the prefill attention once read its accumulator on a barrier parity two phases ahead, a few runs in a hundred).
    for again in range(40):
        runner = ModelRunner(model, num_blocks=700, block_size=16, max_requests=102)
        for r in seqs:
            runner.begin(r)
        for lo in range(0, 100, 25):
            runner.step([StepEntry(r, seqs[r][:-1]) for r in range(lo, lo + 25)])
        runner.step([StepEntry(100, seqs[100][:100])])
        assert np.array_equal(runner.step(entries).float().cpu().numpy(), out), f"run {again} differs from the first"


# ---------------------------------------------------------------------------------------------------
# positions in the thousands
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_one_request_carried_past_position_8000(head_dim, dtype, tmp_path):
    """Portions of 2,048 tokens up to position 8,000, then 40 tokens one by one, with the llama3 frequency bands
    of the large models (original length 8,192, factor 32): the rotation's angles at positions in the thousands
    and block tables hundreds of pages wide, against the plain implementation on the same GPU."""
    from nanospec_b200.config import Llama3RopeScaling, LlamaConfig
    from nanospec_b200.engine import ModelRunner, StepEntry
    from nanospec_b200.weights import write_random_model

    dt = DTYPES[dtype]
    heads = 256 // head_dim
    cfg_t = LlamaConfig(vocab_size=503, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=heads,
                        num_key_value_heads=max(1, heads // 2), head_dim=head_dim, rms_norm_eps=1e-5, rope_theta=500000.0,
                        max_position_embeddings=16384, rope_scaling=Llama3RopeScaling(32.0, 1.0, 4.0, 8192))
    write_random_model(tmp_path, cfg_t, seed=head_dim)
    cfg, w = plain_on_gpu(tmp_path)
    model = load(tmp_path, dt)
    ids = random_ids(8040, 503, seed=77)
    want_all = plain.plain_forward(cfg, w, ids).cpu().numpy()
    runner = ModelRunner(model, num_blocks=-(-len(ids) // 16), block_size=16, max_requests=2)
    runner.begin(0)
    got, places, at = [], [], 0
    while at < 8000:
        n = min(2048, 8000 - at)
        want = sorted({0, 1, n // 2, n - 2, n - 1})
        got.append(runner.step([StepEntry(0, ids[at: at + n], want)]).float().cpu().numpy())
        places += [at + p for p in want]
        at += n
    for p in range(8000, len(ids)):
        got.append(runner.step([StepEntry(0, ids[p: p + 1], [0])]).float().cpu().numpy())
        places.append(p)
    assert max(len(runner.manager.table(0, 0)), 0) == 503
    check_rows(np.concatenate(got), want_all[places], dt, f"head_dim {head_dim} {dtype}, positions up to {places[-1]}")
    runner.end(0)
    runner.manager.check()


# ---------------------------------------------------------------------------------------------------
# the head in chunks, the phase timers, preemption in bfloat16
# ---------------------------------------------------------------------------------------------------
def test_head_in_chunks_smaller_than_the_sampled_rows_and_phase_timers(tiny_folders):
    cfg, w = plain.read_folder(tiny_folders["B"])
    model = load(tiny_folders["B"], torch.float32)
    prompts = [random_ids(n, cfg["vocab"], seed=40 + n) for n in (3, 11, 20, 7, 30)]
    want = [plain.plain_greedy(cfg, w, p, 6)[0] for p in prompts]
    eng = engine(model, num_blocks=64, block_size=8, cuda_graphs=False, head_chunk=2, profile=True, max_admit=8)
    assert eng.generate(prompts, params(max_tokens=6)) == want  # 5 sampled rows in chunks of 2, 2 and 1
    assert set(eng.prof) >= {"forward", "score"}
    assert len(eng.prof["forward"]) == eng.steps and all(t > 0 for t in eng.prof["forward"] + eng.prof["score"])
    # a mixed-temperature batch through the same chunks
    sp = [params(max_tokens=5, temperature=0.9, seed=i) for i in range(5)]
    a = engine(model, num_blocks=64, block_size=8, cuda_graphs=False, head_chunk=2, max_admit=8).generate(prompts, sp)
    b = engine(model, num_blocks=64, block_size=8, cuda_graphs=False, head_chunk=256, max_admit=8).generate(prompts, sp)
    assert a == b


def test_preemption_in_bfloat16(tiny_folders):
    from test_engine_gpu import assert_tokens_match

    cfg, w = plain.read_folder(tiny_folders["B"])
    prompts = [random_ids(n, cfg["vocab"], seed=50 + n) for n in (1, 9, 40, 100)]
    toks, rows = zip(*(plain.plain_greedy(cfg, w, p, 16) for p in prompts))
    model = load(tiny_folders["B"], torch.bfloat16)
    eng = engine(model, num_blocks=20, block_size=8, admission="optimistic", cuda_graphs=True, prefill_chunk=32)
    got = eng.generate(prompts, params(max_tokens=16))
    assert_tokens_match(got, list(toks), list(rows), torch.bfloat16, "optimistic admission in bfloat16")
    assert eng.sched.preempted_total > 0
    eng.cache.check()
    assert eng.cache.free_pages() == [20]


# ---------------------------------------------------------------------------------------------------
# pages are handed out again, and the logits do not care
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_replay_really_uses_pages_again(dtype, tiny_folders):
    from test_replay_gpu import plain_logits, sequences

    name = "B"
    seqs, prompts = sequences(name)
    steps = trace_mixed(seqs, prompts, max_live=4)
    page = TINY[name]["page"]
    model = load(tiny_folders[name], DTYPES[dtype])
    results, pages, runner = replay_in_process(model, steps, num_blocks=peak_tokens(steps) // page, block_size=page)
    shared = [(a, b) for a in pages for b in pages if a < b and pages[a] & pages[b]]
    assert len(shared) >= 3, "the pool is as small as the trace's peak: later requests must get earlier ones' pages"
    assert runner.manager.free_pages() == [peak_tokens(steps) // page]
    check(collect(steps, results, seqs), plain_logits(name, tiny_folders[name]), dtype, f"in-process mixed {dtype}")


# ---------------------------------------------------------------------------------------------------
# a bounded wait that runs out
# ---------------------------------------------------------------------------------------------------
def test_a_bounded_wait_runs_out_and_is_reported():
    """The kernels' waits on mbarriers are bounded; one that runs out records a code that the engine reads.  Here
    the wait itself is shown, in a kernel of one block with nothing in flight whose barrier nobody arrives at
    (csrc/wait_probe.cu), with a limit of a millisecond: it gives up, the error is raised with its text, the flag
    is cleared, and the next kernel on the stream is correct."""
    from nanospec_b200 import ops

    dev = torch.device("cuda", torch.cuda.current_device())
    ops.check_kernel_errors(dev)  # nothing pending
    t0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0[0].record()
    completed = ops.wait_probe(dev, limit_ns=1_000_000)
    t0[1].record()
    torch.cuda.synchronize()
    assert completed is False
    assert t0[0].elapsed_time(t0[1]) < 1000.0  # milliseconds: the limit given, not the two seconds of the production kernels
    with pytest.raises(ops.KernelError, match="gave up waiting on an mbarrier.*wait probe.*code 31"):
        ops.check_kernel_errors(dev)
    ops.check_kernel_errors(dev)  # the flag was cleared by the check that raised
    x = torch.randn(8, 256, device="cuda").to(torch.bfloat16)
    wt = torch.randn(384, 256, device="cuda").to(torch.bfloat16)
    out = torch.empty(8, 384, dtype=torch.bfloat16, device="cuda")
    assert ops.linear_tensor_core(x, wt, out)
    torch.testing.assert_close(out.float(), x.float() @ wt.float().T, rtol=2e-2, atol=2e-2)
    ops.check_kernel_errors(dev)
    with pytest.raises(ops.KernelError, match="limit"):
        ops.wait_probe(dev, limit_ns=5_000_000_000)  # limits beyond a second are refused


# ---------------------------------------------------------------------------------------------------
# a mixer with state under CUDA graphs
# ---------------------------------------------------------------------------------------------------
def test_toy_state_mixer_addressed_on_the_device_runs_under_graphs(tmp_path):
    """The contract for state under graphs: `lane.state[ctx.state_slot[b]]` on the device, padding rows pointing
    at the scratch slot.  A toy mixer (running mean of its inputs, as in test_parts_gpu.py) written with index
    operations only - no host value read in `forward` - is registered from here, run through `Engine.generate`
    with graphs and equals the eager run and a plain statement of the same arithmetic."""
    import dataclasses

    from nanospec_b200.architectures.llama import llama_recipe
    from nanospec_b200.config import Architecture, LlamaConfig, PartSpec, register_architecture
    from nanospec_b200.parts import Part, StateNeed, WeightSpec, register_part
    from nanospec_b200.weights import write_random_model

    @register_part("mixer", "toy_running_mean_on_device")
    class RunningMeanOnDevice(Part):
        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.hidden = spec["hidden"]

        def weight_specs(self):
            return {"mix.weight": WeightSpec((self.hidden, self.hidden))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"]

        def cache_need(self):
            return None

        def state_need(self):
            return StateNeed((self.hidden + 1,), torch.float32)

        def forward(self, x, ctx, lane, writes=True):
            H, N = self.hidden, x.shape[0]
            req = ctx.token_req.long()                      # -1 on padding rows
            pad = req < 0
            b = req.clamp(min=0)
            slot = torch.where(pad, torch.full_like(b, lane.state.shape[0] - 1), ctx.state_slot.long()[b])
            first = torch.where(pad, torch.arange(N, device=x.device), ctx.qo_indptr.long()[b])  # the request's first row
            xs = torch.where(pad[:, None], torch.zeros_like(x), x).float()
            cs = xs.cumsum(0)
            before = torch.where((first > 0)[:, None], cs[(first - 1).clamp(min=0)], torch.zeros_like(cs))
            st = lane.state[slot]
            sums = st[:, :H] + cs - before
            counts = st[:, H] + (torch.arange(N, device=x.device) - first + 1).float()
            out = ctx.buffer("branch", H)
            out.copy_(((sums / counts[:, None]).to(x.dtype)) @ self.w.T)
            # the state after a request's last row stays; the other rows' go to the scratch slot
            last = torch.ones(N, dtype=torch.bool, device=x.device)
            last[:-1] = req[1:] != req[:-1]
            keep = torch.where(last | pad, slot, torch.full_like(slot, lane.state.shape[0] - 1))
            lane.state.index_copy_(0, keep, torch.cat([sums, counts[:, None]], dim=1))
            return out

    def recipe(cfg):
        r = llama_recipe(cfg)
        toy = dataclasses.replace(r.layers[1], mixer=PartSpec("toy_running_mean_on_device", {"hidden": cfg.hidden_size}),
                                  names={**r.layers[1].names, "mixer": "toy."})
        return dataclasses.replace(r, architecture="ToyDeviceStateForCausalLM", layers=(r.layers[0], toy))

    register_architecture(Architecture("ToyDeviceStateForCausalLM", "toy-device-state-test", LlamaConfig.from_hf, recipe))
    cfg_t = LlamaConfig(vocab_size=120, hidden_size=40, intermediate_size=56, num_hidden_layers=2, num_attention_heads=5,
                        num_key_value_heads=5, head_dim=8, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=96)
    hf = cfg_t.to_hf()
    hf["architectures"] = ["ToyDeviceStateForCausalLM"]
    write_random_model(tmp_path, hf, seed=6)
    model = load(tmp_path, torch.float32)
    pcfg, w = plain.read_folder(tmp_path)

    def plain_logits(ids):
        positions = torch.arange(len(ids))
        x = w["model.embed_tokens.weight"][torch.tensor(ids)]
        x = plain.plain_layer(x, w, 0, pcfg, positions, plain.plain_inv_freq(8, 10000.0, None))
        p = "model.layers.1."
        h = plain.plain_rmsnorm(x, w[p + "input_layernorm.weight"], pcfg["eps"])
        x = x + (h.cumsum(0) / torch.arange(1, len(ids) + 1)[:, None]) @ w[p + "toy.mix.weight"].T
        x = x + plain.plain_mlp(plain.plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], pcfg["eps"]), w, p + "mlp.")
        return plain.plain_rmsnorm(x, w["model.norm.weight"], pcfg["eps"]) @ w["lm_head.weight"].T

    prompts = [random_ids(n, 120, seed=n) for n in (9, 4, 12, 2, 7)]
    limits = [12, 5, 9, 3, 7]  # requests end one after another: slots are given back and taken again, buckets shrink
    plist = [params(max_tokens=n) for n in limits]
    outs = {}
    for graphs in (True, False):
        eng = engine(model, num_blocks=64, block_size=4, cuda_graphs=graphs, prefill_chunk=5, max_running=3, max_admit=2,
                     record_logits=True)
        reqs = [eng.add(p, s) for p, s in zip(prompts, plist)]
        while eng.sched.has_work:
            eng.step()
        outs[graphs] = reqs
        if graphs:
            assert eng.graphs.replays > 5
        eng.cache.check()
    for a, b, prompt in zip(outs[True], outs[False], prompts):
        assert a.out_tokens == b.out_tokens
        want = plain_logits(list(prompt) + a.out_tokens[:-1])[len(prompt) - 1:]
        torch.testing.assert_close(torch.stack(a.step_logits), want, rtol=3e-5, atol=3e-6)
        torch.testing.assert_close(torch.stack(b.step_logits), want, rtol=3e-5, atol=3e-6)


# ---------------------------------------------------------------------------------------------------
# the command line on the GPU
# ---------------------------------------------------------------------------------------------------
def _cli(*args: str, stdin: str | None = None) -> str:
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    proc = subprocess.run([sys.executable, "-m", "nanospec_b200", *args], capture_output=True, text=True, input=stdin,
                          env=env, cwd=str(ROOT), timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return proc.stdout


def test_command_line_generate_and_bench(tiny_folders):
    """`python -m nanospec_b200 generate` and `bench` as a user runs them (the reference's manner:
    bench/run.py:162-177): the printed output ids are the plain implementation's greedy tokens, and the lines that
    `bench` prints fold into a table."""
    folder = str(tiny_folders["B"])
    cfg, w = plain.read_folder(folder)
    out = _cli("generate", "--model", folder, "--dtype", "float32", "--block-size", "8", "--prompt-lens", "9", "40",
               "--prompt-ids", "5 17 3", "--max-tokens", "8", "--prefill-chunk", "16")
    rows = [json.loads(line) for line in out.splitlines() if line.startswith("{")]
    g = torch.Generator().manual_seed(0)
    prompts = [[5, 17, 3]] + [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (9, 40)]
    assert [r["prompt_len"] for r in rows[:3]] == [3, 9, 40]
    for r, p in zip(rows[:3], prompts):
        assert r["output_ids"] == plain.plain_greedy(cfg, w, p, 8)[0]
    assert rows[3]["out_tokens"] == 24 and rows[3]["requests"] == 3
    env_out = subprocess.run([sys.executable, "-m", "nanospec_b200", "bench", "--dtype", "float32", "--block-size", "8", "--bs", "1", "2",
                              "--runs", "1", "--prompts", "3", "--prompt-len", "12", "--max-tokens", "6"],
                             capture_output=True, text=True, cwd=str(ROOT), timeout=600,
                             env=dict(os.environ, PYTHONPATH=str(ROOT), NANOSPEC_MODEL=folder))  # the folder from the environment
    assert env_out.returncode == 0, env_out.stderr[-2000:]
    lines = [json.loads(line) for line in env_out.stdout.splitlines() if line.startswith("{")]
    assert [(r["bs"], r["out_tokens"]) for r in lines] == [(1, 18), (2, 18)]
    assert all(r["tok_s"] > 0 and abs(r["tpot_ms"] - 1000 * r["bs"] / r["tok_s"]) < 0.05 * r["tpot_ms"] for r in lines)
    table = _cli("table", stdin=env_out.stdout)
    assert table.splitlines()[0].startswith("| engine |") and "| nanospec_b200 | nospec | 2 |" in table


# ---------------------------------------------------------------------------------------------------
# layers with different needs in one model: all keys beside a window of them
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_a_window_beside_layers_with_all_keys_through_the_engine(dtype, tmp_path):
    """A recipe registered from here: layer 0 reads every key, layers 1 and 2 the last 24 only.  The two kinds form
    two cache groups with pools and block tables of their own; the windowed group gives pages back while its
    requests run (they decode far past what it could hold otherwise) and hands them out again.  Generation through
    graphs and through eager steps, portions of 32, every step's logits against the plain implementation with the
    same windows."""
    import dataclasses

    from nanospec_b200.architectures.llama import llama_recipe
    from nanospec_b200.cache import RELEASED
    from nanospec_b200.config import Architecture, LlamaConfig, PartSpec, register_architecture, registered_architectures
    from nanospec_b200.weights import write_random_model

    window = 24

    def recipe(cfg):
        r = llama_recipe(cfg)
        layers = list(r.layers)
        for i in (1, 2):
            m = layers[i].mixer
            layers[i] = dataclasses.replace(layers[i], mixer=PartSpec(m.kind, {**m.params, "window": window}))
        return dataclasses.replace(r, architecture="WindowedForCausalLM", layers=tuple(layers))

    if "WindowedForCausalLM" not in registered_architectures():  # the test runs once per dtype
        register_architecture(Architecture("WindowedForCausalLM", "windowed-test", LlamaConfig.from_hf, recipe))
    cfg_t = LlamaConfig(vocab_size=700, hidden_size=256, intermediate_size=384, num_hidden_layers=3, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=256)
    hf = cfg_t.to_hf()
    hf["architectures"] = ["WindowedForCausalLM"]
    write_random_model(tmp_path, hf, seed=12)
    pcfg, w = plain.read_folder(tmp_path)
    dt = DTYPES[dtype]
    model = load(tmp_path, dt)
    assert [n[0].window for n in model.lane_needs()] == [0, window, window]

    def plain_logits(ids):
        positions = torch.arange(len(ids))
        inv = plain.plain_inv_freq(64, 10000.0, None)
        x = w["model.embed_tokens.weight"][torch.tensor(ids)]
        for i in range(3):
            p = f"model.layers.{i}."
            h = plain.plain_rmsnorm(x, w[p + "input_layernorm.weight"], pcfg["eps"])
            x = x + plain.plain_attention_block(h, w, p + "self_attn.", pcfg, positions, inv, window if i else 0)
            x = x + plain.plain_mlp(plain.plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], pcfg["eps"]), w, p + "mlp.")
        return plain.plain_rmsnorm(x, w["model.norm.weight"], pcfg["eps"]) @ w["lm_head.weight"].T

    prompts = [random_ids(n, 700, seed=60 + n) for n in (50, 9, 120)]
    limits = [70, 40, 30]
    page = 8
    for graphs in (True, False):
        eng = engine(model, num_blocks=40, block_size=page, cuda_graphs=graphs, record_logits=True, prefill_chunk=32, max_admit=2)
        assert len(eng.cache.groups) == 2 and eng.cache.groups[1].spec.window == window
        reqs = [eng.add(p, params(max_tokens=n)) for p, n in zip(prompts, limits)]
        most_held, released_seen = 0, False
        while eng.sched.has_work:
            eng.step()
            eng.cache.check()
            for r in reqs:
                if r.state == "running":
                    most_held = max(most_held, eng.cache.held_pages(r.id)[1])
                    released_seen |= RELEASED in eng.cache.table(1, r.id)
        # window - 1 + a portion of 32 positions, and one page more for alignment: far less than the 19 pages of 150 positions
        assert most_held <= -(-(window - 1 + 32) // page) + 1 and released_seen
        assert eng.cache.free_pages() == [40, 40] and eng.cache.live == []
        for i, (req, prompt) in enumerate(zip(reqs, prompts)):
            ids = list(prompt) + req.out_tokens
            want = plain_logits(ids[:-1])[len(prompt) - 1:].numpy()
            check_rows(torch.stack(req.step_logits).numpy(), want, dt, f"windowed layers, {dtype}, graphs={graphs}, request {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_at_real_widths_keeps_every_logit(dtype, wide_folders):
    """Optimistic admission on a pool that is far too small (dozens of preemptions), heads of 64 at real widths,
    graphs on: requests are dropped and recomputed from their prompt plus what they had emitted.  Every step's
    logits against the plain implementation over the request's own tokens; in float32 the tokens are those of an
    engine with room for everybody."""
    dt = DTYPES[dtype]
    folder = wide_folders["wide64"]
    vocab = WIDE["wide64"].vocab_size
    cfg, w = plain_on_gpu(folder)
    model = load(folder, dt)
    prompts = [random_ids(10 + (53 * i) % 200, vocab, seed=300 + i) for i in range(10)]
    plist = [params(max_tokens=16 + (i * 7) % 20) for i in range(10)]
    eng = engine(model, num_blocks=24, block_size=16, admission="optimistic", prefill_chunk=64, record_logits=True)
    reqs = [eng.add(p, s) for p, s in zip(prompts, plist)]
    while eng.sched.has_work:
        eng.step()
        eng.cache.check()
    assert eng.sched.preempted_total >= 10 and eng.cache.free_pages() == [24] and eng.cache.live == []
    check_teacher_forced(reqs, prompts, cfg, w, dt, f"preemption at real widths, {dtype}")
    if dtype == "float32":
        roomy = engine(model, num_blocks=400, block_size=16, cuda_graphs=False, lookahead=False)
        assert roomy.generate(prompts, plist) == [r.out_tokens for r in reqs]


# ---------------------------------------------------------------------------------------------------
# random schedules
# ---------------------------------------------------------------------------------------------------
def test_random_engine_options_and_arrivals_give_the_plain_tokens(tiny_folders):
    """Sixty random combinations of everything the scheduler can be told - pool size down to what the largest request
    needs, page-sized to whole-prompt portions, a token budget down to one, one to eight live requests, both
    admission policies, graphs, launching ahead, the head in chunks, requests that arrive later - on the three tiny
    models in float32, where the tokens must be the plain implementation's whatever the schedule."""
    import random

    models = {n: load(tiny_folders[n], torch.float32) for n in TINY}
    plains = {n: plain.read_folder(tiny_folders[n]) for n in TINY}
    known: dict[tuple, list[int]] = {}

    def greedy(name, prompt, n):
        key = (name, tuple(prompt))
        if key not in known or len(known[key]) < n:
            known[key] = plain.plain_greedy(*plains[name], prompt, n)[0]
        return known[key][:n]

    for it in range(60):
        rng = random.Random(7000 + it)
        name = rng.choice(list(TINY))
        cfg, page = TINY[name]["config"], TINY[name]["page"]
        max_pos = cfg.max_position_embeddings
        reqs = []
        for _ in range(rng.randint(1, 9)):
            plen = rng.choice([1, 2, 3, rng.randint(1, 40), rng.randint(1, min(120, max_pos - 20))])
            reqs.append((random_ids(plen, cfg.vocab_size, seed=rng.randint(0, 50)), rng.randint(1, min(14, max_pos - plen))))
        need = max(-(-(len(p) + n) // page) for p, n in reqs)
        kw = dict(num_blocks=rng.choice([need, need + 1, need + rng.randint(0, 10), 200]), block_size=page,
                  cuda_graphs=rng.random() < 0.6, lookahead=rng.random() < 0.7, max_admit=rng.choice([1, 2, 32]),
                  max_running=rng.choice([None, 1, 2, 3, 8]), prefill_chunk=rng.choice([1, 2, 5, 16, 2048]),
                  max_step_tokens=rng.choice([1, 3, 9, 40, 8192]), admission=rng.choice(["reserve", "optimistic"]),
                  head_chunk=rng.choice([1, 3, 256]), capture_at_start=rng.random() < 0.3)
        eng = engine(models[name], **kw)
        rs = [eng.add(p, params(max_tokens=n)) for p, n in reqs]
        late = []
        if rng.random() < 0.5 and len(rs) > 2:  # the last two arrive after three steps
            late = rs[-2:]
            for r in late:
                eng.sched.waiting.remove(r)
        steps = 0
        while eng.sched.has_work or late:
            if late and (steps >= 3 or not eng.sched.has_work):
                for r in late:
                    eng.sched.add(r)
                late = []
            eng.step()
            steps += 1
            eng.cache.check()
            assert steps < 5000, (it, kw)
        assert [r.out_tokens for r in rs] == [greedy(name, p, n) for p, n in reqs], (it, name, kw, [(len(p), n) for p, n in reqs])
        assert eng.cache.live == [] and all(f == kw["num_blocks"] for f in eng.cache.free_pages()), (it, kw)


@pytest.mark.parametrize("name", ["wide64", "wide128"])
def test_random_cuts_at_real_widths(name, wide_folders):
    """Fifteen random traces per model in bfloat16: one to six requests of 1 to 700 tokens, every step a random choice of
    who takes part and of portion sizes that sit on and beside every tile edge of the kernels (1, 2, 3, 15-17, 31-33, 63-65,
    127-129, 255-257, 300), pages of 8 to 64, pools with two pages to spare; the logits of every position against the
    plain implementation."""
    import random

    from nanospec_b200.engine import ModelRunner, StepEntry

    sizes = [1, 1, 1, 2, 3, 15, 16, 17, 31, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300]
    vocab = WIDE[name].vocab_size
    cfg, w = plain_on_gpu(wide_folders[name])
    model = load(wide_folders[name], torch.bfloat16)
    for it in range(15):
        rng = random.Random(4200 + it)
        lens = [rng.choice([1, 2, 5, 64, 65, 129, rng.randint(1, 400), rng.randint(200, 700)]) for _ in range(rng.randint(1, 6))]
        seqs = {r: random_ids(n, vocab, seed=rng.randint(0, 10 ** 6)) for r, n in enumerate(lens)}
        page = rng.choice([8, 16, 32, 64])
        runner = ModelRunner(model, num_blocks=sum(-(-n // page) for n in lens) + 2, block_size=page, max_requests=8)
        for r in seqs:
            runner.begin(r)
        pos = {r: 0 for r in seqs}
        got = {r: [] for r in seqs}
        first = True
        while any(pos[r] < lens[r] for r in seqs):
            entries = [(r, pos[r], min(rng.choice(sizes), lens[r] - pos[r])) for r in seqs
                       if pos[r] < lens[r] and (first or rng.random() >= 0.2)]
            if not entries:
                continue
            first = False
            out = runner.step([StepEntry(r, seqs[r][a: a + n], list(range(n))) for r, a, n in entries]).float().cpu().numpy()
            row = 0
            for r, a, n in entries:
                got[r].append(out[row: row + n])
                row += n
                pos[r] = a + n
        runner.manager.check()
        for r, ids in seqs.items():
            check_rows(np.concatenate(got[r]), plain.plain_forward(cfg, w, ids).cpu().numpy(), torch.bfloat16,
                       f"{name}, trace {it}, pages of {page}, request {r} of {lens[r]} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,heads,kv", [(16, 6, 3), (48, 9, 3), (80, 4, 1), (96, 6, 2), (112, 3, 3), (64, 24, 2), (160, 2, 1), (256, 2, 2)])
def test_whole_models_at_other_head_sizes(d, heads, kv, dtype, tmp_path):
    """Head sizes in steps of 16 from 16 to 128 (the tensor-core attention kernels: a group of 12 query heads per kv head
    among them), and 160 and 256 (the exact kernel), as whole two-layer models with widths that are no power of two:
    random cuts with pages of 4 to 32, every position's logits against the plain implementation."""
    import random

    from nanospec_b200.config import Llama3RopeScaling, LlamaConfig
    from nanospec_b200.engine import ModelRunner, StepEntry
    from nanospec_b200.weights import write_random_model

    cfg_t = LlamaConfig(vocab_size=503 + d, hidden_size=16 * ((heads * d // 2) // 16 + 3), intermediate_size=24 * (d // 8 + 5),
                        num_hidden_layers=2, num_attention_heads=heads, num_key_value_heads=kv, head_dim=d, rms_norm_eps=1e-5,
                        rope_theta=50000.0, max_position_embeddings=1024,
                        rope_scaling=Llama3RopeScaling(4.0, 1.0, 4.0, 128) if d % 32 else None)
    write_random_model(tmp_path, cfg_t, seed=4)
    cfg, w = plain_on_gpu(tmp_path)
    dt = DTYPES[dtype]
    model = load(tmp_path, dt)
    sizes = [1, 1, 2, 3, 15, 17, 33, 63, 64, 65, 127, 129, 200]
    for it in range(3):
        rng = random.Random(100 * d + it)
        lens = [rng.choice([1, 2, 65, 129, rng.randint(1, 300), rng.randint(200, 600)]) for _ in range(rng.randint(1, 5))]
        seqs = {r: random_ids(n, cfg_t.vocab_size, seed=rng.randint(0, 10 ** 6)) for r, n in enumerate(lens)}
        page = rng.choice([4, 8, 16, 32])
        runner = ModelRunner(model, num_blocks=sum(-(-n // page) for n in lens) + 2, block_size=page, max_requests=8)
        for r in seqs:
            runner.begin(r)
        pos = {r: 0 for r in seqs}
        got = {r: [] for r in seqs}
        while any(pos[r] < lens[r] for r in seqs):
            entries = [(r, pos[r], min(rng.choice(sizes), lens[r] - pos[r])) for r in seqs if pos[r] < lens[r] and rng.random() > 0.15]
            if not entries:
                continue
            out = runner.step([StepEntry(r, seqs[r][a: a + n], list(range(n))) for r, a, n in entries]).float().cpu().numpy()
            row = 0
            for r, a, n in entries:
                got[r].append(out[row: row + n])
                row += n
                pos[r] = a + n
        runner.manager.check()
        for r, ids in seqs.items():
            check_rows(np.concatenate(got[r]), plain.plain_forward(cfg, w, ids).cpu().numpy(), dt,
                       f"head size {d}, {heads} heads over {kv}, {dtype}, trace {it}, request {r}")


def test_weights_replaced_in_place_at_real_widths(wide_folders, tmp_path):
    """The packed tensors of the fused kernels (q/k/v in one matrix, gate and up rows alternating in runs of 64, a head
    tied to the embedding) are rebuilt from checkpoint tensors and copied in place: an engine whose weights were
    replaced gives, through the graphs it captured before, the tokens of an engine loaded from the other folder."""
    from nanospec_b200.weights import write_random_model

    write_random_model(tmp_path, WIDE["wide64"], seed=77)
    _, w2 = plain.read_folder(tmp_path)
    vocab = WIDE["wide64"].vocab_size
    prompts = [random_ids(n, vocab, seed=640 + n) for n in (9, 70, 33)]
    swapped = engine(load(wide_folders["wide64"], torch.bfloat16), num_blocks=64, block_size=16)
    first = swapped.generate(prompts, params(max_tokens=6))
    swapped.update_weights({k: v for k, v in w2.items() if k != "lm_head.weight"})  # the head follows the embedding
    fresh = engine(load(tmp_path, torch.bfloat16), num_blocks=64, block_size=16)
    want = fresh.generate(prompts, params(max_tokens=10))
    assert swapped.generate(prompts, params(max_tokens=10)) == want and [w[:6] for w in want] != first

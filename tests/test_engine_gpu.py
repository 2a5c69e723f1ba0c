"""Generation through the Python entry point on the GPU: greedy tokens against the plain
implementation, batching, portions, CUDA graphs, small pools, preemption, temperature
sampling with seeds, long decoding, and the first tokens of a sequence.  In the manner of the
reference's tests/test_correctness.py, test_batching.py, test_graphs.py and
test_sampling.py:170-191, on tiny random models instead of a downloaded checkpoint."""

from __future__ import annotations

import pytest
import torch

import plain_llama as plain
from conftest import TINY, random_ids

pytestmark = pytest.mark.gpu


def load(folder, dtype):
    from nanospec_b200 import load_model
    return load_model(folder, device="cuda", dtype=dtype)


def engine(model, **kw):
    from nanospec_b200 import Engine, EngineConfig
    kw.setdefault("num_blocks", 128)
    return Engine(model, EngineConfig(**kw))


def params(**kw):
    from nanospec_b200 import SamplingParams
    return SamplingParams(**kw)


_plain = {}


def plain_model(name, folder):
    if name not in _plain:
        _plain[name] = plain.read_folder(folder)
    return _plain[name]


def assert_tokens_match(got, want, want_logits, dtype, what):
    """float32: strictly equal.  bfloat16: the reference's rule (tests/conftest.py:30-55 there):
    a divergence is allowed only where the exact logits of our token lie within 8 bf16 ulps of
    the row maximum of the best one; after it the sequences are different texts."""
    for i, (a, b) in enumerate(zip(got, want)):
        if a == b:
            continue
        assert dtype != torch.float32, f"{what}: request {i}: {a} != {b}"
        j = next(k for k in range(min(len(a), len(b))) if a[k] != b[k])
        z = want_logits[i][j]
        gap = float(z.max() - z[a[j]])
        assert gap <= 8 * 2.0 ** -7 * float(z.abs().max()), f"{what}: request {i} step {j}: gap {gap}"


PROMPT_LENS = {"A": [5, 17, 33, 64], "B": [1, 9, 40, 100], "C": [3, 50, 77]}


@pytest.fixture(scope="module")
def oracle(tiny_folders):
    out = {}
    for name, lens in PROMPT_LENS.items():
        cfg, w = plain_model(name, tiny_folders[name])
        prompts = [random_ids(n, cfg["vocab"], seed=50 + n) for n in lens]
        toks, rows = zip(*(plain.plain_greedy(cfg, w, p, 16) for p in prompts))
        out[name] = (prompts, list(toks), list(rows))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_matches_plain(name, dtype, tiny_folders, oracle):
    prompts, want, rows = oracle[name]
    model = load(tiny_folders[name], dtype)
    page = TINY[name]["page"]
    for what, kw in {
        "one at a time": dict(max_running=1, cuda_graphs=False),
        "all at once": dict(max_admit=32, cuda_graphs=False),
        "staggered, portions of 7": dict(max_admit=1, prefill_chunk=7, cuda_graphs=False),
        "budget of 24 tokens a step": dict(max_step_tokens=24, prefill_chunk=16, cuda_graphs=False),
        "graphs": dict(max_admit=2, cuda_graphs=True),
    }.items():
        eng = engine(model, block_size=page, **kw)
        got = eng.generate(prompts, params(max_tokens=16))
        assert_tokens_match(got, want, rows, dtype, f"{name} {dtype} {what}")
        eng.cache.check()
        assert eng.cache.free_pages() == [128] and not eng.cache.live
        if kw.get("cuda_graphs"):
            assert eng.graphs.replays > 0


def test_graph_and_eager_logits_agree_while_the_batch_crosses_buckets(tiny_folders):
    """Per-step logits with graphs against eager, as tests/test_graphs.py:43-72 in the reference."""
    model = load(tiny_folders["B"], torch.float32)
    cfg = TINY["B"]["config"]
    prompts = [random_ids(3 + 2 * i, cfg.vocab_size, seed=i) for i in range(9)]
    sp = [params(max_tokens=4 + 3 * i) for i in range(9)]  # requests finish one after another: 9 -> 1 live
    outs = {}
    for graphs in (False, True):
        eng = engine(model, block_size=8, cuda_graphs=graphs, record_logits=True, max_admit=3)
        reqs = [eng.add(p, s) for p, s in zip(prompts, sp)]
        while eng.sched.has_work:
            eng.step()
        outs[graphs] = reqs
        if graphs:
            assert set(eng.graphs.buckets) >= {1, 2, 4, 8, 16}
    for a, b in zip(outs[False], outs[True]):
        assert a.out_tokens == b.out_tokens
        for za, zb in zip(a.step_logits, b.step_logits):
            assert torch.equal(za, zb)  # float32: the same kernels in the same order, with or without a graph


def test_small_pool_throttles_and_finish_order_differs_from_arrival(tiny_folders, oracle):
    prompts, want, rows = oracle["A"]
    model = load(tiny_folders["A"], torch.float32)
    # 64 + 16 - 1 positions need 5 pages; with 7 pages the long request runs with at most one short one
    eng = engine(model, num_blocks=7, block_size=16, cuda_graphs=False)
    sp = [params(max_tokens=16), params(max_tokens=3), params(max_tokens=16), params(max_tokens=16)]
    reqs = [eng.add(p, s) for p, s in zip(prompts, sp)]
    order = []
    while eng.sched.has_work:
        order += [r.id for r in eng.step()]
        eng.cache.check()
    assert [r.out_tokens for r in reqs] == [w[: s.max_tokens] for w, s in zip(want, sp)]
    assert order != sorted(order) and sorted(order) == [0, 1, 2, 3]
    assert eng.sched.preempted_total == 0


@pytest.mark.parametrize("dtype", [torch.float32])
def test_optimistic_admission_preempts_and_still_gives_the_same_tokens(dtype, tiny_folders, oracle):
    prompts, want, rows = oracle["B"]
    model = load(tiny_folders["B"], dtype)
    # the four requests need 2 + 3 + 7 + 15 pages of 8 in the end; 20 pages force a preemption
    eng = engine(model, num_blocks=20, block_size=8, admission="optimistic", cuda_graphs=True, prefill_chunk=32)
    got = eng.generate(prompts, params(max_tokens=16))
    assert got == want
    assert eng.sched.preempted_total > 0
    eng.cache.check()
    assert eng.cache.free_pages() == [20]


def test_temperature_sampling_is_reproducible_and_independent_of_the_batch(tiny_folders):
    cfg_t = TINY["B"]["config"]
    cfg, w = plain_model("B", tiny_folders["B"])
    model = load(tiny_folders["B"], torch.float32)
    prompts = [random_ids(n, cfg_t.vocab_size, seed=70 + n) for n in (1, 9, 40, 100, 130, 250)]
    sps = [params(max_tokens=12, temperature=0.8, seed=3 + i, logprobs=True) for i in range(len(prompts))]
    runs = []
    for kw in (dict(max_running=1, cuda_graphs=False), dict(max_admit=2, prefill_chunk=32, cuda_graphs=False),
               dict(max_admit=6, prefill_chunk=32, cuda_graphs=True)):
        eng = engine(model, num_blocks=256, block_size=8, **kw)
        reqs = [eng.add(p, s) for p, s in zip(prompts, sps)]
        while eng.sched.has_work:
            eng.step()
        runs.append(reqs)
    for a, b, c in zip(*runs):
        assert a.out_tokens == b.out_tokens == c.out_tokens
    # against the plain implementation, fed the same uniforms from the same seeded generator
    for i, r in enumerate(runs[0]):
        gen = torch.Generator().manual_seed(3 + i)
        ids = list(prompts[i])
        for t, info in zip(r.out_tokens, r.logprobs):
            u = float(torch.rand(1, generator=gen))
            z = plain.plain_forward(cfg, w, ids)[-1]
            lp = plain.plain_process(z, 0.8)
            want = plain.plain_draw(lp, u)
            if want != t:  # only a cdf boundary within rounding may flip a draw
                cdf = lp.exp().cumsum(-1)
                assert abs(float(cdf[min(t, want)]) - u * float(cdf[-1])) < 1e-5, (i, t, want)
            assert abs(info.sample_logprob - float(lp[t])) < 1e-4
            assert abs(info.logprob - float(z.log_softmax(-1)[t])) < 1e-4
            ids.append(t)
    # greedy and sampled requests share a batch; top-k / top-p run through the same path
    eng = engine(model, num_blocks=256, block_size=8, cuda_graphs=True)
    mixed = [params(max_tokens=8), params(max_tokens=8, temperature=1.0, top_k=5, seed=1),
             params(max_tokens=8, temperature=0.7, top_p=0.5, seed=2)]
    out = eng.generate(prompts[1:4], mixed)
    assert out[0] == plain.plain_greedy(cfg, w, prompts[1], 8)[0]
    eng2 = engine(model, num_blocks=256, block_size=8, cuda_graphs=False, max_running=1)
    assert eng2.generate(prompts[1:4], mixed) == out


def test_long_decoding_and_first_tokens(tiny_folders):
    """A one-token prompt decoded to the model's position limit, token for token against the
    plain implementation; every page edge and the rescaled rotary bands are crossed."""
    name = "B"
    cfg, w = plain_model(name, tiny_folders[name])
    model = load(tiny_folders[name], torch.float32)
    n_new = 300
    eng = engine(model, num_blocks=64, block_size=8, cuda_graphs=True, record_logits=True)
    req = eng.add([17], params(max_tokens=n_new))
    while eng.sched.has_work:
        eng.step()
    ids = [17] + req.out_tokens
    z = plain.plain_forward(cfg, w, ids[:-1])  # teacher-forced on the engine's own tokens
    got = torch.stack(req.step_logits)
    err = (got - z).abs().max(dim=1).values
    assert float(err.max()) < 2e-5, f"first wrong step {int((err >= 2e-5).nonzero()[0])}"
    top2 = z.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 1e-4
    assert torch.equal(torch.tensor(req.out_tokens)[clear], z.argmax(-1)[clear])
    # the very first positions, each alone
    for n in (1, 2, 3):
        e = engine(model, num_blocks=8, block_size=8, cuda_graphs=False, record_logits=True)
        r = e.add(ids[:n], params(max_tokens=1))
        e.step()
        assert float((r.step_logits[0] - z[n - 1]).abs().max()) < 2e-5


def test_eos_stops_and_is_kept(tiny_folders, tmp_path):
    import json
    import shutil

    cfg, w = plain_model("A", tiny_folders["A"])
    prompt = random_ids(12, cfg["vocab"], seed=9)
    greedy, _ = plain.plain_greedy(cfg, w, prompt, 8)
    folder = tmp_path / "with_eos"
    shutil.copytree(tiny_folders["A"], folder)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [greedy[3], 9999]}))
    model = load(folder, torch.float32)
    eng = engine(model, cuda_graphs=False)
    stop = greedy.index(greedy[3]) + 1
    assert eng.generate([prompt], params(max_tokens=8)) == [greedy[:stop]]
    assert eng.generate([prompt], params(max_tokens=8, ignore_eos=True)) == [greedy]


def test_a_step_launched_ahead_changes_nothing(tiny_folders, tmp_path):
    """Steps are launched before their predecessor's tokens have reached the host.  Requests
    that end meanwhile (an end token, their own max_tokens) make the extra step run in vain: the
    tokens are those of an engine that never looks ahead, with and without graphs, and every page
    comes back."""
    import json
    import shutil

    cfg, w = plain_model("B", tiny_folders["B"])
    prompts = [random_ids(n, cfg["vocab"], seed=70 + n) for n in (6, 19, 33, 2)]
    greedy = [plain.plain_greedy(cfg, w, p, 14)[0] for p in prompts]
    folder = tmp_path / "ends"
    shutil.copytree(tiny_folders["B"], folder)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [greedy[1][5]]}))
    model = load(folder, torch.float32)
    limits = [14, 14, 9, 3]
    plist = [params(max_tokens=n) for n in limits]
    want = []
    for g, n in zip(greedy, limits):
        g = g[:n]
        stop = next((i + 1 for i, t in enumerate(g) if t == greedy[1][5]), len(g))
        want.append(g[:stop])
    assert len(want[1]) <= 6 and len({len(x) for x in want}) >= 3   # they end at different steps
    for kw in (dict(cuda_graphs=True, lookahead=True), dict(cuda_graphs=True, lookahead=False),
               dict(cuda_graphs=False, lookahead=True), dict(cuda_graphs=False, lookahead=False),
               # portions of prompts beside decode tokens, launched ahead as well
               dict(cuda_graphs=False, lookahead=True, prefill_chunk=7, max_admit=1),
               dict(cuda_graphs=True, lookahead=True, prefill_chunk=5, max_step_tokens=9),
               dict(cuda_graphs=False, lookahead=False, prefill_chunk=7, max_admit=1),
               # a queue: four requests through two slots, so that steps which admit somebody are launched ahead too
               dict(cuda_graphs=True, lookahead=True, max_running=2), dict(cuda_graphs=False, lookahead=True, max_running=2, prefill_chunk=7),
               dict(cuda_graphs=True, lookahead=False, max_running=2),
               # portions of one token: a prompt's last token, which the host knows, shares a graph step launched ahead with
               # decode tokens that are still on the device
               dict(cuda_graphs=True, lookahead=True, prefill_chunk=1, max_admit=1)):
        eng = engine(model, num_blocks=40, block_size=8, **kw)
        assert eng.generate(prompts, plist) == want, kw
        eng.cache.check()
        assert eng.cache.live == [] and all(f == 40 for f in eng.cache.free_pages()), kw
        if kw.get("lookahead") and not kw["cuda_graphs"]:
            assert eng.launched_ahead > 0, kw
        if kw.get("lookahead") and kw.get("max_running") == 2:
            assert eng.launched_ahead >= eng.steps - 4, kw   # nearly every step, those that admit the third and fourth included


def test_a_step_launched_for_requests_that_are_gone_costs_no_call(tiny_folders):
    """Requests taken away while a step launched ahead for them is in flight: the next call of `step`
    does not spend itself on reading that step, it runs what is there to run."""
    cfg, w = plain_model("A", tiny_folders["A"])
    model = load(tiny_folders["A"], torch.float32)
    for graphs in (True, False):
        eng = engine(model, cuda_graphs=graphs)
        olds = [eng.add(random_ids(n, cfg["vocab"], seed=n), params(max_tokens=50, ignore_eos=True)) for n in (4, 9)]
        for _ in range(5):
            eng.step()
        assert eng.launched_ahead > 0 and eng._inflight is not None
        for r in olds:
            eng.sched.finish(r)
        prompt = random_ids(11, cfg["vocab"], seed=3)
        new = eng.add(prompt, params(max_tokens=1))
        assert eng.step() == [new] and new.out_tokens == plain.plain_greedy(cfg, w, prompt, 1)[0]
        eng.cache.check()
        assert eng.cache.live == []


def test_errors_are_loud(tiny_folders):
    from nanospec_b200.engine import RequestTooLarge
    model = load(tiny_folders["A"], torch.float32)
    eng = engine(model, num_blocks=2, block_size=16, cuda_graphs=False)
    with pytest.raises(RequestTooLarge):
        eng.add(list(range(40)), params(max_tokens=8))
    eng = engine(model, cuda_graphs=False)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.add([1, 2, 999], params(max_tokens=2))
    with pytest.raises(ValueError, match="positions"):
        eng.add([1] * 250, params(max_tokens=8))
    cpu_model = __import__("nanospec_b200").load_model(tiny_folders["A"], device="cpu", dtype=torch.float32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        engine(cpu_model)


def test_weights_replaced_in_place_restart_the_running_requests(tiny_folders, tmp_path):
    """`Engine.update_weights` (the reference's engine/engine.py:167-176): new weights are copied into the tensors the
    kernels and the captured graphs point at, and every running request is recomputed from its prompt plus what it has
    emitted.  After the swap the tokens are those of the plain implementation with the new weights over that longer prompt."""
    from nanospec_b200.weights import WeightError, write_random_model

    name = "B"
    cfg_t = TINY[name]["config"]
    other = tmp_path / "other"
    write_random_model(other, cfg_t, seed=909)
    cfg1, w1 = plain_model(name, tiny_folders[name])
    cfg2, w2 = plain.read_folder(other)
    new_state = {k: v for k, v in w2.items()}
    prompts = [random_ids(n, cfg_t.vocab_size, seed=80 + n) for n in (7, 30, 2)]
    for graphs in (True, False):
        model = load(tiny_folders[name], torch.float32)
        eng = engine(model, num_blocks=64, block_size=8, cuda_graphs=graphs)
        reqs = [eng.add(p, params(max_tokens=12)) for p in prompts]
        for _ in range(5):
            eng.step()
        before = [list(r.out_tokens) for r in reqs]
        assert all(0 < len(b) < 12 for b in before) and eng._inflight is not None
        for p, b in zip(prompts, before):
            assert b == plain.plain_greedy(cfg1, w1, p, len(b))[0]
        eng.update_weights(new_state)
        assert eng._inflight is None and [r.state for r in reqs] == ["waiting"] * 3
        while eng.sched.has_work:
            eng.step()
        for p, b, r in zip(prompts, before, reqs):
            assert r.out_tokens[: len(b)] == b
            assert r.out_tokens[len(b):] == plain.plain_greedy(cfg2, w2, p + b, 12 - len(b))[0], graphs
        eng.cache.check()
        # a part's packed tensors go together; unknown names and wrong shapes are refused before anything is written
        with pytest.raises(WeightError, match="replaced together"):
            eng.update_weights({"model.layers.0.self_attn.q_proj.weight": w2["model.layers.0.self_attn.q_proj.weight"]})
        with pytest.raises(WeightError, match="unexpected"):
            eng.update_weights({"model.layers.9.mlp.down_proj.weight": w2["model.layers.0.mlp.down_proj.weight"]})
        with pytest.raises(WeightError, match="wrong shape"):
            eng.update_weights({"model.norm.weight": torch.ones(3)})
        eng.update_weights({"model.norm.weight": w1["model.norm.weight"]})  # a part alone

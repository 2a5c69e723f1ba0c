"""The parts of a layer, each alone against its plain statement, and the generality of their
assembly: a recipe whose order names a layer twice and lets a run read another run's cache,
and a toy mixer with state of its own that is defined here, registered, built from a model
folder and stepped - without a change to the framework's files."""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_llama as plain
from conftest import random_ids

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


class _Shell:
    """Just enough of a model for ModelRunner to build step contexts for parts under test."""

    bound = True
    device = DEV
    vocab_size = 1000

    def __init__(self, dtype, needs, max_positions=512):
        from types import SimpleNamespace
        self.dtype = dtype
        self._needs = needs
        self.recipe = SimpleNamespace(max_positions=max_positions)

    def lane_needs(self):
        return self._needs


def context(dtype, needs, entries, page=8, num_blocks=64):
    """entries: list of (req_id, n_tokens); returns (runner, ctx)."""
    from nanospec_b200.engine import ModelRunner, StepEntry
    runner = ModelRunner(_Shell(dtype, needs), num_blocks, page, 8)
    for rid, _ in entries:
        runner.begin(rid)
    ctx, _, _ = runner.build_context([StepEntry(rid, [1] * n) for rid, n in entries])
    return runner, ctx


def step_context(runner, entries):
    from nanospec_b200.engine import StepEntry
    return runner.build_context([StepEntry(rid, [1] * n) for rid, n in entries])[0]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part_alone(dtype):
    from nanospec_b200.config import PartSpec
    from nanospec_b200.parts import build_part
    norm = build_part("norm", PartSpec("rmsnorm", {"hidden": 200, "eps": 1e-4}), dtype, DEV)
    assert norm.weight_specs()["weight"].shape == (200,)
    g = torch.Generator().manual_seed(1)
    gain = 1 + 0.1 * torch.randn(200, generator=g)
    norm.bind({"weight": gain.to(DEV)})
    _, ctx = context(dtype, [], [(0, 7)])
    resid = torch.randn(7, 200, generator=g).to(DEV)
    pending = torch.randn(7, 200, generator=g).to(dtype).to(DEV)
    want_resid = resid + pending.float()
    out = norm.add_norm(resid, pending, ctx)
    torch.testing.assert_close(resid, want_resid, rtol=0, atol=0)
    torch.testing.assert_close(out.float().cpu(), plain.plain_rmsnorm(want_resid.cpu(), gain, 1e-4), **tol(dtype))


def test_position_part_alone_matches_the_reference_frequencies():
    from nanospec_b200.config import PartSpec
    from nanospec_b200.parts import build_part
    scaling = {"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
    for d, theta, sc in ((128, 500000.0, scaling), (64, 500000.0, scaling), (16, 10000.0, None)):
        rope = build_part("position", PartSpec("rope", {"head_dim": d, "theta": theta, "scaling": sc}), torch.float32, DEV)
        assert torch.equal(rope.inv_freq_host, plain.plain_inv_freq(d, theta, sc))  # bit for bit


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,d,hidden,window", [(6, 3, 16, 80, 0), (4, 1, 32, 96, 0), (4, 2, 16, 64, 11),
                                                            (4, 2, 64, 128, 0), (8, 4, 32, 256, 9)])  # the last two: rotation in the projection's epilogue
def test_attention_mixer_alone_over_two_steps(dtype, heads, kv_heads, d, hidden, window):
    """The mixer on its own cache lane: a portion, then the rest, against whole-sequence attention."""
    from nanospec_b200.config import PartSpec
    from nanospec_b200.parts import build_part
    pos = PartSpec("rope", {"head_dim": d, "theta": 10000.0, "scaling": None})
    spec = PartSpec("gqa_attention", {"hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": d,
                                      "window": window, "position": pos})
    mixer = build_part("mixer", spec, dtype, DEV)
    g = torch.Generator().manual_seed(heads)
    weights = {n: (torch.randn(s.shape, generator=g) * 0.1).to(dtype) for n, s in mixer.weight_specs().items()}
    mixer.bind({n: t.to(DEV) for n, t in weights.items()})
    S, cut = 37, 21
    x = torch.randn(S, hidden, generator=g).to(dtype)
    wf = {"p." + n: t.float() for n, t in weights.items()}
    cfg = {"heads": heads, "kv_heads": kv_heads, "head_dim": d}
    want = plain.plain_attention_block(x.float(), wf, "p.", cfg, torch.arange(S), plain.plain_inv_freq(d, 10000.0, None), window)
    runner, ctx = context(dtype, [(mixer.cache_need(), mixer.state_need())], [(0, cut)])
    assert mixer.cache_need().window == window
    y1 = mixer.forward(x[:cut].to(DEV).contiguous(), ctx, ctx.lanes[0]).clone()
    runner.manager.trim(0)
    ctx = step_context(runner, [(0, S - cut)])
    y2 = mixer.forward(x[cut:].to(DEV).contiguous(), ctx, ctx.lanes[0])
    torch.testing.assert_close(torch.cat([y1, y2]).float().cpu(), want, **tol(dtype))


def test_blocks_fold_their_norms_into_the_products_of_a_short_step():
    """Two blocks in bfloat16 on a step of 5 tokens: the products take over the residual sums and the
    norms (the second block is handed a RowScaled), and stream and output agree with the norm kernels."""
    from nanospec_b200 import ops
    from nanospec_b200.config import LayerSpec, PartSpec
    from nanospec_b200.parts import build_block
    hidden, heads, kvh, d, inter = 256, 4, 2, 64, 384
    pos = PartSpec("rope", {"head_dim": d, "theta": 10000.0, "scaling": None})
    layer = LayerSpec(mixer=PartSpec("gqa_attention", {"hidden": hidden, "heads": heads, "kv_heads": kvh, "head_dim": d,
                                                       "window": 0, "position": pos}),
                      feed_forward=PartSpec("swiglu", {"hidden": hidden, "intermediate": inter}),
                      norm=PartSpec("rmsnorm", {"hidden": hidden, "eps": 1e-5}), prefix="l.", block="prenorm",
                      names={"mixer": "a.", "feed_forward": "f.", "norm_mixer": "n1.", "norm_feed_forward": "n2."})
    g = torch.Generator().manual_seed(11)
    blocks = [build_block(layer, torch.bfloat16, DEV) for _ in range(2)]
    for b in blocks:
        for part in b.parts().values():
            part.bind({n: ((1 + 0.1 * torch.randn(s.shape, generator=g)) if s.init == "gain" else
                           torch.randn(s.shape, generator=g) * 0.05).to(torch.float32 if s.rule == "float32" else torch.bfloat16).to(DEV)
                       for n, s in part.weight_specs().items()})
    need = [(blocks[0].mixer.cache_need(), None)]
    x0 = torch.randn(5, hidden, generator=g)
    outs = {}
    for fuse in (True, False):
        ops.FUSE_NORM = fuse
        try:
            _, ctx = context(torch.bfloat16, need + need, [(0, 5)])
            resid = x0.clone().to(DEV)
            resid, pending = blocks[0].forward(resid, None, ctx, ctx.lanes[0], True, follow=blocks[1])
            assert isinstance(pending, ops.RowScaled) == fuse
            resid, pending = blocks[1].forward(resid, pending, ctx, ctx.lanes[1], True)
            assert isinstance(pending, torch.Tensor)
            outs[fuse] = (resid.clone(), pending.float().clone())
        finally:
            ops.FUSE_NORM = True
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    torch.testing.assert_close(outs[True][0], outs[False][0], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(outs[True][1], outs[False][1], rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part_alone(dtype):
    from nanospec_b200.config import PartSpec
    from nanospec_b200.parts import build_part
    ff = build_part("feed_forward", PartSpec("swiglu", {"hidden": 72, "intermediate": 200}), dtype, DEV)
    g = torch.Generator().manual_seed(2)
    weights = {n: (torch.randn(s.shape, generator=g) * 0.1).to(dtype) for n, s in ff.weight_specs().items()}
    ff.bind({n: t.to(DEV) for n, t in weights.items()})
    x = torch.randn(9, 72, generator=g).to(dtype)
    _, ctx = context(dtype, [], [(0, 9)])
    got = ff.forward(x.to(DEV), ctx)
    want = plain.plain_mlp(x.float(), {"p." + n: t.float() for n, t in weights.items()}, "p.")
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype))


# ---------------------------------------------------------------------------------------
# the order of layers is data
# ---------------------------------------------------------------------------------------
def test_a_layer_named_twice_and_a_run_that_reads_another_runs_cache(tmp_path):
    import dataclasses

    from nanospec_b200.architectures.llama import llama_recipe
    from nanospec_b200.config import Architecture, LlamaConfig, Run, register_architecture
    from nanospec_b200.engine import ModelRunner, StepEntry
    from nanospec_b200.weights import load_model, write_random_model

    def recipe(cfg):
        r = llama_recipe(cfg)
        # layer 0, layer 1, layer 0 again on a lane of its own, layer 1 again reading the keys
        # and values that its first run wrote
        return dataclasses.replace(r, architecture="TwiceForCausalLM",
                                   order=(Run(0, 0), Run(1, 1), Run(0, 2), Run(1, 1, writes=False)))

    register_architecture(Architecture("TwiceForCausalLM", "twice-test", LlamaConfig.from_hf, recipe))
    cfg = LlamaConfig(vocab_size=97, hidden_size=48, intermediate_size=80, num_hidden_layers=2, num_attention_heads=3,
                      num_key_value_heads=1, head_dim=16, rms_norm_eps=1e-5, rope_theta=10000.0,
                      max_position_embeddings=128)
    hf = cfg.to_hf()
    hf["architectures"] = ["TwiceForCausalLM"]
    write_random_model(tmp_path, hf, seed=4)
    model = load_model(tmp_path, device="cuda", dtype=torch.float32)
    assert [n[0].head_dim for n in model.lane_needs()] == [16, 16, 16]

    pcfg, w = plain.read_folder(tmp_path)
    ids = random_ids(29, 97, seed=8)
    inv = plain.plain_inv_freq(16, 10000.0, None)
    positions = torch.arange(len(ids))

    def layer(x, i, kv=None):
        p = f"model.layers.{i}."
        h = plain.plain_rmsnorm(x, w[p + "input_layernorm.weight"], pcfg["eps"])
        S = x.shape[0]
        a = p + "self_attn."
        q = plain.plain_rope((h @ w[a + "q_proj.weight"].T).view(S, 3, 16), positions, inv)
        if kv is None:
            k = plain.plain_rope((h @ w[a + "k_proj.weight"].T).view(S, 1, 16), positions, inv)
            v = (h @ w[a + "v_proj.weight"].T).view(S, 1, 16)
        else:
            k, v = kv
        x = x + plain.plain_attention(q, k, v).reshape(S, -1) @ w[a + "o_proj.weight"].T
        x = x + plain.plain_mlp(plain.plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], pcfg["eps"]), w, p + "mlp.")
        return x, (k, v)

    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    x, _ = layer(x, 0)
    x, kv1 = layer(x, 1)
    x, _ = layer(x, 0)
    x, _ = layer(x, 1, kv=kv1)
    want = plain.plain_rmsnorm(x, w["model.norm.weight"], pcfg["eps"]) @ w["lm_head.weight"].T

    runner = ModelRunner(model, num_blocks=16, block_size=4, max_requests=2)
    runner.begin(0)
    got = [runner.step([StepEntry(0, ids[:13], list(range(13)))]), runner.step([StepEntry(0, ids[13:27], list(range(14)))]),
           runner.step([StepEntry(0, ids[27:28], [0])]), runner.step([StepEntry(0, ids[28:], [0])])]
    torch.testing.assert_close(torch.cat(got).cpu(), want, rtol=2e-5, atol=2e-6)


# ---------------------------------------------------------------------------------------
# a toy mixer with state of its own
# ---------------------------------------------------------------------------------------
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    """The toy mixer keeps, per request, the running sum of its inputs and a count (fixed-size
    state, no pages): y_t = W * mean(x_0..x_t).  It is defined here with plain torch
    operations, registered under a new name, put into a recipe beside an attention layer,
    written to and loaded from a model folder, and stepped in different cuts and through
    `Engine.generate`; requests that end give their state slot back and the next request
    finds it zeroed."""
    from nanospec_b200 import Engine, EngineConfig, SamplingParams
    from nanospec_b200.architectures.llama import llama_recipe
    from nanospec_b200.config import Architecture, LayerSpec, LlamaConfig, PartSpec, register_architecture
    from nanospec_b200.engine import ModelRunner, StepEntry
    from nanospec_b200.parts import Part, StateNeed, WeightSpec, register_part
    from nanospec_b200.weights import load_model, write_random_model
    import dataclasses

    @register_part("mixer", "toy_running_mean")
    class RunningMean(Part):
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
            out = ctx.buffer("branch", self.hidden)
            start = 0
            for b, n in enumerate(ctx.q_lens):
                slot = ctx.state_slots_host[b]
                st = lane.state[slot]
                xs = x[start:start + n].float()
                sums = st[: self.hidden] + xs.cumsum(0)
                counts = st[self.hidden] + torch.arange(1, n + 1, device=x.device)
                mean = (sums / counts[:, None]).to(x.dtype)
                out[start:start + n] = mean @ self.w.T
                st[: self.hidden] = sums[-1]
                st[self.hidden] = counts[-1]
                start += n
            return out

    def recipe(cfg):
        r = llama_recipe(cfg)
        toy = dataclasses.replace(r.layers[1], mixer=PartSpec("toy_running_mean", {"hidden": cfg.hidden_size}),
                                  names={**r.layers[1].names, "mixer": "toy."})
        return dataclasses.replace(r, architecture="ToyForCausalLM", layers=(r.layers[0], toy))

    register_architecture(Architecture("ToyForCausalLM", "toy-test", LlamaConfig.from_hf, recipe))
    cfg = LlamaConfig(vocab_size=120, hidden_size=40, intermediate_size=56, num_hidden_layers=2, num_attention_heads=5,
                      num_key_value_heads=5, head_dim=8, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=96)
    hf = cfg.to_hf()
    hf["architectures"] = ["ToyForCausalLM"]
    write_random_model(tmp_path, hf, seed=6)
    assert "model.layers.1.toy.mix.weight" in json.dumps(sorted(plain.read_folder(tmp_path)[1]))
    model = load_model(tmp_path, device="cuda", dtype=torch.float32)
    needs = model.lane_needs()
    assert needs[0][0] is not None and needs[0][1] is None and needs[1][0] is None and needs[1][1].shape == (41,)

    pcfg, w = plain.read_folder(tmp_path)

    def plain_logits(ids):
        positions = torch.arange(len(ids))
        x = w["model.embed_tokens.weight"][torch.tensor(ids)]
        x = plain.plain_layer(x, w, 0, pcfg, positions, plain.plain_inv_freq(8, 10000.0, None))
        p = "model.layers.1."
        h = plain.plain_rmsnorm(x, w[p + "input_layernorm.weight"], pcfg["eps"])
        mean = h.cumsum(0) / torch.arange(1, len(ids) + 1)[:, None]
        x = x + mean @ w[p + "toy.mix.weight"].T
        x = x + plain.plain_mlp(plain.plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], pcfg["eps"]), w, p + "mlp.")
        return plain.plain_rmsnorm(x, w["model.norm.weight"], pcfg["eps"]) @ w["lm_head.weight"].T

    seqs = {0: random_ids(30, 120, seed=1), 1: random_ids(17, 120, seed=2), 2: random_ids(22, 120, seed=3)}
    runner = ModelRunner(model, num_blocks=24, block_size=4, max_requests=2)
    got = {r: [] for r in seqs}

    def run(entries):
        out = runner.step([StepEntry(r, seqs[r][a:b], list(range(b - a))) for r, a, b in entries])
        row = 0
        for r, a, b in entries:
            got[r].append(out[row: row + b - a].cpu())
            row += b - a

    runner.begin(0), runner.begin(1)
    run([(0, 0, 11), (1, 0, 2)])
    run([(1, 2, 3), (0, 11, 13)])
    run([(0, 13, 30), (1, 3, 17)])
    runner.end(1)
    runner.begin(2)  # takes the slot that request 1 held: it must start from zero state
    run([(2, 0, 9)])
    run([(2, 9, 22)])
    runner.end(0), runner.end(2)
    runner.manager.check()
    for r, ids in seqs.items():
        torch.testing.assert_close(torch.cat(got[r]), plain_logits(ids), rtol=3e-5, atol=3e-6)

    # and through the entry point (no graphs: the toy mixer reads host values)
    eng = Engine(model, EngineConfig(num_blocks=32, block_size=4, cuda_graphs=False, prefill_chunk=7, max_running=2))
    prompts = [seqs[0][:9], seqs[1][:4], seqs[2][:12]]
    outs = eng.generate(prompts, SamplingParams(max_tokens=5))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for t in o:
            z = plain_logits(ids)[-1]
            top = z.topk(2).values
            assert t == int(z.argmax()) or float(top[0] - top[1]) < 1e-5
            ids.append(t)


def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path):
    """Two more parts defined here and registered from outside the package: a feed-forward that routes every
    token to one of three experts (router logits in float32), and a position encoding that rotates interleaved
    pairs (2i, 2i+1) instead of halves.  A model folder that names them is written, loaded, stepped in
    portions beside another request, and compared with a plain statement of the same arithmetic."""
    from nanospec_b200 import ops
    from nanospec_b200.architectures.llama import llama_recipe
    from nanospec_b200.config import Architecture, LlamaConfig, PartSpec, register_architecture
    from nanospec_b200.engine import ModelRunner, StepEntry
    from nanospec_b200.parts import Part, WeightSpec, register_part
    from nanospec_b200.weights import load_model, write_random_model
    import dataclasses

    @register_part("feed_forward", "toy_top1_experts")
    class Top1Experts(Part):
        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.hidden, self.inter, self.experts = spec["hidden"], spec["intermediate"], spec["experts"]

        def weight_specs(self):
            specs = {"router.weight": WeightSpec((self.experts, self.hidden), rule="float32", std=0.5)}
            for e in range(self.experts):
                specs[f"experts.{e}.up.weight"] = WeightSpec((self.inter, self.hidden), std=0.1)
                specs[f"experts.{e}.down.weight"] = WeightSpec((self.hidden, self.inter), std=0.1)
            return specs

        def bind(self, tensors):
            self.w = tensors

        def forward(self, x, ctx):
            logits = x.float() @ self.w["router.weight"].T          # router logits in float32
            prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
            out = ctx.buffer("branch", self.hidden)
            out.zero_()
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(x[rows] @ self.w[f"experts.{e}.up.weight"].T)
                    y = (h @ self.w[f"experts.{e}.down.weight"].T).float() * prob[rows, None]
                    out[rows] = y.to(out.dtype)
            return out

    @register_part("position", "toy_interleaved_rotary")
    class InterleavedRotary(Part):
        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            d = spec["head_dim"]
            self.freq = (1.0 / (spec["theta"] ** (torch.arange(0, d, 2).float() / d))).to(device)

        def rotate_and_store(self, qkv, ctx, lane, nq, nkv, head_dim, writes):
            ang = ctx.positions.float()[:, None] * self.freq[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            qk = qkv[:, : (nq + nkv) * head_dim].view(-1, nq + nkv, head_dim // 2, 2).float()
            a, b = qk[..., 0], qk[..., 1]
            rot = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1)
            qkv[:, : (nq + nkv) * head_dim] = rot.reshape(qkv.shape[0], -1).to(qkv.dtype)
            if writes:
                ops.kv_store(qkv, ctx, lane, nq, nkv, head_dim)

    heads, kvh, d, hidden, inter, experts = 4, 2, 16, 48, 40, 3

    def recipe(cfg):
        r = llama_recipe(cfg)
        mixer = r.layers[0].mixer
        toy_pos = PartSpec("toy_interleaved_rotary", {"head_dim": d, "theta": 100.0})
        l0 = dataclasses.replace(r.layers[0], mixer=PartSpec(mixer.kind, {**mixer.params, "position": toy_pos}))
        l1 = dataclasses.replace(r.layers[1], feed_forward=PartSpec("toy_top1_experts", {"hidden": hidden, "intermediate": inter,
                                                                                         "experts": experts}),
                                 names={**r.layers[1].names, "feed_forward": "moe."})
        return dataclasses.replace(r, architecture="ToyRoutedForCausalLM", layers=(l0, l1))

    register_architecture(Architecture("ToyRoutedForCausalLM", "toy-routed-test", LlamaConfig.from_hf, recipe))
    cfg = LlamaConfig(vocab_size=90, hidden_size=hidden, intermediate_size=64, num_hidden_layers=2, num_attention_heads=heads,
                      num_key_value_heads=kvh, head_dim=d, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=64)
    hf = cfg.to_hf()
    hf["architectures"] = ["ToyRoutedForCausalLM"]
    write_random_model(tmp_path, hf, seed=9)
    pcfg, w = plain.read_folder(tmp_path)
    assert "model.layers.1.moe.experts.2.down.weight" in w and w["model.layers.1.moe.router.weight"].dtype == torch.float32
    model = load_model(tmp_path, device="cuda", dtype=torch.float32)

    def plain_logits(ids):
        S = len(ids)
        positions = torch.arange(S)
        x = w["model.embed_tokens.weight"][torch.tensor(ids)].float()
        # layer 0: attention with interleaved rotary, the usual feed-forward
        p = "model.layers.0."
        h = plain.plain_rmsnorm(x, w[p + "input_layernorm.weight"], pcfg["eps"])
        q = (h @ w[p + "self_attn.q_proj.weight"].float().T).view(S, heads, d)
        k = (h @ w[p + "self_attn.k_proj.weight"].float().T).view(S, kvh, d)
        v = (h @ w[p + "self_attn.v_proj.weight"].float().T).view(S, kvh, d)
        ang = positions.float()[:, None] * (1.0 / (100.0 ** (torch.arange(0, d, 2).float() / d)))[None, :]

        def rot(t):
            a, b = t[..., 0::2], t[..., 1::2]
            c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
            return torch.stack([a * c - b * s, b * c + a * s], dim=-1).reshape(t.shape)

        att = plain.plain_attention(rot(q), rot(k), v).reshape(S, heads * d)
        x = x + att @ w[p + "self_attn.o_proj.weight"].float().T
        x = x + plain.plain_mlp(plain.plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], pcfg["eps"]), w, p + "mlp.")
        # layer 1: the usual attention, the routed feed-forward
        p = "model.layers.1."
        h = plain.plain_rmsnorm(x, w[p + "input_layernorm.weight"], pcfg["eps"])
        x = x + plain.plain_attention_block(h, w, p + "self_attn.", {"heads": heads, "kv_heads": kvh, "head_dim": d}, positions,
                                            plain.plain_inv_freq(d, 10000.0, None))
        h = plain.plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], pcfg["eps"])
        prob, choice = torch.softmax(h @ w[p + "moe.router.weight"].T, dim=-1).max(dim=-1)
        y = torch.zeros_like(x)
        for e in range(experts):
            rows = (choice == e).nonzero().flatten()
            up, down = w[p + f"moe.experts.{e}.up.weight"].float(), w[p + f"moe.experts.{e}.down.weight"].float()
            y[rows] = (torch.relu(h[rows] @ up.T) @ down.T) * prob[rows, None]
        x = x + y
        return plain.plain_rmsnorm(x, w["model.norm.weight"], pcfg["eps"]) @ w["lm_head.weight"].float().T, choice

    seqs = {0: random_ids(27, 90, seed=4), 1: random_ids(15, 90, seed=5)}
    runner = ModelRunner(model, num_blocks=24, block_size=4, max_requests=2)
    got = {r: [] for r in seqs}

    def run(entries):
        out = runner.step([StepEntry(r, seqs[r][a:b], list(range(b - a))) for r, a, b in entries])
        row = 0
        for r, a, b in entries:
            got[r].append(out[row: row + b - a].float().cpu())
            row += b - a

    runner.begin(0), runner.begin(1)
    run([(0, 0, 9), (1, 0, 2)])
    run([(1, 2, 3), (0, 9, 11)])
    run([(0, 11, 27), (1, 3, 15)])
    runner.end(0), runner.end(1)
    runner.manager.check()
    for r, ids in seqs.items():
        want, choice = plain_logits(ids)
        assert len(set(choice.tolist())) > 1  # the router really sends tokens to different experts
        torch.testing.assert_close(torch.cat(got[r]), want, rtol=3e-5, atol=3e-6)


def test_toy_norm_and_toy_block_arrangement(tmp_path):
    """The last two kinds of part, defined here and registered from outside the package: a norm that centres
    its input and has a bias (it cannot be folded into a product: it has no `sink`), and a block arrangement
    that feeds one norm's output to the mixer and to the feed-forward side by side, x + mixer(n(x)) + ff(n(x)).
    A model whose first layer is that block, whose second layer is the usual one and whose final norm is the toy
    norm is written, loaded, stepped in portions and generated from through graphs, against a plain statement."""
    import dataclasses

    from nanospec_b200 import Engine, EngineConfig, SamplingParams
    from nanospec_b200.architectures.llama import llama_recipe
    from nanospec_b200.config import Architecture, LlamaConfig, PartSpec, register_architecture, registered_architectures
    from nanospec_b200.engine import ModelRunner, StepEntry
    from nanospec_b200.parts import Part, WeightSpec, build_part, register_part
    from nanospec_b200.weights import load_model, write_random_model

    @register_part("norm", "toy_centred")
    class CentredNorm(Part):
        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.hidden, self.eps = spec["hidden"], spec["eps"]

        def weight_specs(self):
            return {"weight": WeightSpec((self.hidden,), rule="float32", init="gain"),
                    "bias": WeightSpec((self.hidden,), rule="float32", std=0.1)}

        def bind(self, tensors):
            self.w = tensors

        def add_norm(self, resid, pending, ctx, rows=None, out_name="normed"):
            if rows is None:
                if pending is not None:
                    resid += pending.float()          # the stream takes the branch, in place
                x = resid
            else:                                     # only these rows, the stream untouched
                x = resid[rows.long()] + (pending[rows.long()].float() if pending is not None else 0.0)
            x = x - x.mean(dim=-1, keepdim=True)
            y = x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + self.eps) * self.w["weight"] + self.w["bias"]
            out = ctx.buffer(out_name, self.hidden, rows=x.shape[0])
            out.copy_(y)
            return out

    @register_part("block", "toy_side_by_side")
    class SideBySide:
        def __init__(self, layer, dtype, device):
            self.mixer = build_part("mixer", layer.mixer, dtype, device)
            self.feed_forward = build_part("feed_forward", layer.feed_forward, dtype, device)
            self.norm = build_part("norm", layer.norm, dtype, device)
            self.hidden = layer.norm["hidden"]

        def parts(self):
            return {"norm": self.norm, "mixer": self.mixer, "feed_forward": self.feed_forward}

        def forward(self, resid, pending, ctx, lane, writes=True):
            x = self.norm.add_norm(resid, pending, ctx)
            kept = ctx.buffer("toy_kept_branch", self.hidden)
            kept.copy_(self.mixer.forward(x, ctx, lane, writes))  # the feed-forward's result takes the same buffer
            out = self.feed_forward.forward(x, ctx)
            out += kept
            return resid, out

    heads, kvh, d, hidden, inter, eps = 3, 1, 32, 72, 88, 3e-4
    toy_norm = PartSpec("toy_centred", {"hidden": hidden, "eps": eps})

    def recipe(cfg):
        r = llama_recipe(cfg)
        l0 = dataclasses.replace(r.layers[0], block="toy_side_by_side", norm=toy_norm,
                                 names={"norm": "ln.", "mixer": "self_attn.", "feed_forward": "mlp."})
        return dataclasses.replace(r, architecture="ToySideBySideForCausalLM", layers=(l0, r.layers[1]), final_norm=toy_norm)

    if "ToySideBySideForCausalLM" not in registered_architectures():
        register_architecture(Architecture("ToySideBySideForCausalLM", "toy-side-test", LlamaConfig.from_hf, recipe))
    cfg = LlamaConfig(vocab_size=150, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=2, num_attention_heads=heads,
                      num_key_value_heads=kvh, head_dim=d, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=128)
    hf = cfg.to_hf()
    hf["architectures"] = ["ToySideBySideForCausalLM"]
    write_random_model(tmp_path, hf, seed=12)
    pcfg, w = plain.read_folder(tmp_path)
    assert "model.layers.0.ln.bias" in w and "model.norm.bias" in w and "model.layers.0.input_layernorm.weight" not in w
    inv_freq = plain.plain_inv_freq(d, 10000.0, None)
    shape = {"heads": heads, "kv_heads": kvh, "head_dim": d}

    def centred(x, p):
        x = x - x.mean(dim=-1, keepdim=True)
        return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w[p + "weight"] + w[p + "bias"]

    def plain_logits(ids):
        positions = torch.arange(len(ids))
        x = w["model.embed_tokens.weight"][torch.tensor(ids)].float()
        h = centred(x, "model.layers.0.ln.")
        x = x + plain.plain_attention_block(h, w, "model.layers.0.self_attn.", shape, positions, inv_freq) \
            + plain.plain_mlp(h, w, "model.layers.0.mlp.")
        x = plain.plain_layer(x, w, 1, pcfg, positions, inv_freq)
        return centred(x, "model.norm.") @ w["lm_head.weight"].float().T

    model = load_model(tmp_path, device="cuda", dtype=torch.float32)
    seqs = {0: random_ids(41, 150, seed=21), 1: random_ids(18, 150, seed=22)}
    runner = ModelRunner(model, num_blocks=24, block_size=4, max_requests=2)
    got = {r: [] for r in seqs}

    def run(entries):
        out = runner.step([StepEntry(r, seqs[r][a:b], list(range(b - a))) for r, a, b in entries])
        row = 0
        for r, a, b in entries:
            got[r].append(out[row: row + b - a].float().cpu())
            row += b - a

    runner.begin(0), runner.begin(1)
    run([(0, 0, 13), (1, 0, 2)])
    run([(1, 2, 3), (0, 13, 15)])
    run([(0, 15, 40), (1, 3, 18)])
    run([(0, 40, 41)])
    runner.end(0), runner.end(1)
    runner.manager.check()
    for r, ids in seqs.items():
        torch.testing.assert_close(torch.cat(got[r]), plain_logits(ids), rtol=3e-5, atol=3e-6)
    del runner

    # through the entry point, decode steps replayed from graphs (the toy parts are torch operations on device
    # tensors: they can be captured) and launched ahead, against eager steps and against the plain argmax
    prompts = [seqs[0][:9], seqs[1][:4], seqs[0][5:30]]
    outs = {}
    for graphs in (True, False):
        eng = Engine(model, EngineConfig(num_blocks=64, block_size=4, cuda_graphs=graphs, prefill_chunk=7, max_running=3))
        outs[graphs] = eng.generate(prompts, SamplingParams(max_tokens=6))
        assert not graphs or eng.graphs.replays >= 4
    for graphs in (True, False):
        for p, o in zip(prompts, outs[graphs]):
            ids = list(p)
            for t in o:
                z = plain_logits(ids)[-1]
                top = z.topk(2).values
                assert t == int(z.argmax()) or float(top[0] - top[1]) < 1e-5
                ids.append(t)


def test_toy_embedding_and_toy_head(tmp_path):
    """The two remaining slots: an embedding that scales its rows by sqrt(hidden) and adds a learned offset, and a head
    with a bias whose logits are soft-capped, both defined here.  Through the runner in portions and through
    `Engine.generate` with graphs (head and sampling are inside the graph), against a plain statement."""
    import dataclasses

    from nanospec_b200 import Engine, EngineConfig, SamplingParams, ops
    from nanospec_b200.architectures.llama import llama_recipe
    from nanospec_b200.config import Architecture, LlamaConfig, PartSpec, register_architecture, registered_architectures
    from nanospec_b200.engine import ModelRunner, StepEntry
    from nanospec_b200.parts import Part, WeightSpec, register_part
    from nanospec_b200.weights import load_model, write_random_model

    vocab, hidden, cap = 130, 64, 3.0

    @register_part("embedding", "toy_scaled")
    class ScaledEmbedding(Part):
        def weight_specs(self):
            return {"weight": WeightSpec((vocab, hidden), std=0.05), "offset": WeightSpec((hidden,), rule="float32", std=0.1)}

        def bind(self, tensors):
            self.w = tensors

        def forward(self, ctx):
            resid = ops.embed(self.w["weight"], ctx.token_ids, ctx.buffer("resid", hidden, torch.float32))
            resid.mul_(math.sqrt(hidden)).add_(self.w["offset"])
            return resid

    @register_part("head", "toy_soft_capped")
    class SoftCappedHead(Part):
        def weight_specs(self):
            return {"weight": WeightSpec((vocab, hidden), std=0.3), "bias": WeightSpec((vocab,), rule="float32", std=0.5)}

        def bind(self, tensors):
            self.w = tensors

        def forward(self, h, out=None):
            z = ops.linear(h, self.w["weight"], torch.empty((h.shape[0], vocab), dtype=torch.float32, device=h.device))
            z = cap * torch.tanh((z + self.w["bias"]) / cap)
            if out is None:
                return z
            out.copy_(z)
            return out

    def recipe(cfg):
        r = llama_recipe(cfg)
        return dataclasses.replace(r, architecture="ToyEndsForCausalLM",
                                   embedding=PartSpec("toy_scaled", {"name": "model.embed_tokens"}),
                                   head=PartSpec("toy_soft_capped", {"name": "lm_head"}))

    if "ToyEndsForCausalLM" not in registered_architectures():
        register_architecture(Architecture("ToyEndsForCausalLM", "toy-ends-test", LlamaConfig.from_hf, recipe))
    cfg = LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=80, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=96)
    hf = cfg.to_hf()
    hf["architectures"] = ["ToyEndsForCausalLM"]
    write_random_model(tmp_path, hf, seed=15)
    pcfg, w = plain.read_folder(tmp_path)
    assert w["model.embed_tokens.offset"].dtype == torch.float32 and "lm_head.bias" in w

    def plain_logits(ids):
        positions = torch.arange(len(ids))
        x = w["model.embed_tokens.weight"][torch.tensor(ids)].float() * math.sqrt(hidden) + w["model.embed_tokens.offset"]
        inv_freq = plain.plain_inv_freq(16, 10000.0, None)
        for layer in range(2):
            x = plain.plain_layer(x, w, layer, pcfg, positions, inv_freq)
        z = plain.plain_rmsnorm(x, w["model.norm.weight"], pcfg["eps"]) @ w["lm_head.weight"].float().T + w["lm_head.bias"]
        return cap * torch.tanh(z / cap)

    model = load_model(tmp_path, device="cuda", dtype=torch.float32)
    seqs = {0: random_ids(33, vocab, seed=31), 1: random_ids(12, vocab, seed=32)}
    runner = ModelRunner(model, num_blocks=24, block_size=4, max_requests=2)
    got = {r: [] for r in seqs}
    runner.begin(0), runner.begin(1)
    for entries in ([(0, 0, 10), (1, 0, 3)], [(1, 3, 4), (0, 10, 12)], [(0, 12, 33), (1, 4, 12)]):
        out = runner.step([StepEntry(r, seqs[r][a:b], list(range(b - a))) for r, a, b in entries])
        row = 0
        for r, a, b in entries:
            got[r].append(out[row: row + b - a].float().cpu())
            row += b - a
    runner.end(0), runner.end(1)
    for r, ids in seqs.items():
        torch.testing.assert_close(torch.cat(got[r]), plain_logits(ids), rtol=3e-5, atol=3e-6)
    del runner

    prompts = [seqs[0][:7], seqs[1][:3]]
    for graphs in (True, False):
        eng = Engine(model, EngineConfig(num_blocks=64, block_size=4, cuda_graphs=graphs, max_running=2))
        outs = eng.generate(prompts, SamplingParams(max_tokens=6))
        assert not graphs or eng.graphs.replays >= 4
        for p, o in zip(prompts, outs):
            ids = list(p)
            for t in o:
                z = plain_logits(ids)[-1]
                top = z.topk(2).values
                assert t == int(z.argmax()) or float(top[0] - top[1]) < 1e-5
                ids.append(t)

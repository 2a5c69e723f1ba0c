"""The reference arm of bench.py: the same workloads on the unmodified reference engine.

The reference (ved1beta/nanospec) is a flat tree of pure-Python packages (`engine`, `model`, `kv`,
`sched`, `spec`) that imports from its source root; an unmodified copy of that tree lies under
`baseline/_ref` and is put on `sys.path` here.  Nothing of `nanospec_b200` is imported in this arm.

Its stock path is driven the way its own harness does (bench/run.py:73-86 there): a
`LlamaForCausalLM` in bfloat16 on the GPU with its default attention backend (FlashInfer's paged
wrappers and fused norm / rotation kernels, model/attention.py:46-110), `Engine(model,
EngineConfig(num_blocks, 16, max_admit=min(bs, 8), max_running=bs))` with its CUDA graphs
(engine/graphs.py:171-210), `add` for every prompt, then `step()` while work remains.  The model
is built directly from `LlamaConfig.from_hf(<the benchmark's config.json keys>)` with seeded
N(0, 0.02) weights, since no checkpoint can be fetched; the prompts are seeded uniform-random ids.

If FlashInfer cannot run (it compiles its kernels at first use), the error is quoted and the
reference's other stock path is measured instead and labelled: `SdpaBackend`, `cuda_graphs=False`.
"""

from __future__ import annotations

import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def reference_present() -> str | None:
    """None when the copy of the reference is in place, else what is missing."""
    for rel in ("engine/engine.py", "model/llama.py", "kv/cache.py", "sched/scheduler.py"):
        if not os.path.isfile(os.path.join(REF, rel)):
            return f"baseline/_ref/{rel} is missing: copy the reference's source tree to baseline/_ref"
    return None


def _hf_config(shape: dict, rope: tuple) -> dict:
    cfg = dict(shape)
    cfg["model_type"] = "llama"
    cfg["rope_scaling"] = {"rope_type": "llama3", "factor": rope[0], "low_freq_factor": rope[1], "high_freq_factor": rope[2],
                           "original_max_position_embeddings": rope[3]}
    cfg["tie_word_embeddings"] = False
    return cfg


def _build_model(shape: dict, rope: tuple, backend: str):
    import torch
    from model.attention import SdpaBackend, default_backend
    from model.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig.from_hf(_hf_config(shape, rope))
    dev = torch.device("cuda")
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)  # the loader casts every tensor, norm gains included, to the run's dtype
    try:
        with torch.device("meta"):
            net = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(old)
    g = torch.Generator(device=dev).manual_seed(0)
    state = {}
    for name, p in net.state_dict().items():
        t = torch.empty(p.shape, dtype=torch.bfloat16, device=dev)
        if t.dim() == 2:
            t.normal_(0.0, 0.02, generator=g)
        else:
            t.fill_(1.0)
        state[name] = t
    net.load_state_dict(state, strict=True, assign=True)  # as model/loader.py:68 does
    net.backend = SdpaBackend() if backend == "sdpa" else default_backend(cfg, dev, torch.bfloat16)
    return net.eval()


def _prime(eng, SamplingParams, batch: int, context: int, max_tokens: int, vocab: int, seed: int = 0):
    import torch

    g = torch.Generator().manual_seed(seed)
    reqs = [eng.add(torch.randint(0, vocab, (context - 1,), generator=g).tolist(), SamplingParams(max_tokens, seed=i))
            for i in range(batch)]
    while eng.sched.waiting:
        eng.step()
    return reqs


def _decode_point(net, batch: int, context: int, steps: int, warmup: int, repeats: int, page: int, graphs: bool, sampler_cls):
    """Median over `repeats` of (device ms per step, host seconds per step) for `steps` decode steps of
    `batch` requests that hold `context` tokens each."""
    import torch
    from engine.engine import Engine, EngineConfig
    from sched.scheduler import SamplingParams

    total = warmup + repeats * steps + 16
    num_blocks = batch * (-(-(context + total) // page) + 1) + 8
    eng = Engine(net, EngineConfig(num_blocks, page, max_admit=min(batch, 8), max_running=batch, cuda_graphs=graphs))
    sampler = sampler_cls()
    sampler.start()
    reqs = _prime(eng, SamplingParams, batch, context, total, net.config.vocab_size)
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    sampler.mark()
    dev_ms, host_s = [], []
    for _ in range(repeats):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        a.record()
        for _ in range(steps):
            eng.step()  # host ids -> device, forward (graph replay), head + sampling, tokens back to the host
        b.record()
        torch.cuda.synchronize()
        host_s.append((time.perf_counter() - t0) / steps)
        dev_ms.append(a.elapsed_time(b) / steps)
    clocks = sampler.stop()
    assert all(r.state == "running" for r in reqs)
    del eng
    torch.cuda.empty_cache()
    dev_ms.sort(), host_s.sort()
    return dev_ms[len(dev_ms) // 2], host_s[len(host_s) // 2], (dev_ms[0], dev_ms[-1]), clocks


def _prefill_point(net, tokens: int, page: int, warmup: int, iters: int, graphs: bool) -> float:
    import torch
    from engine.engine import Engine, EngineConfig
    from sched.scheduler import SamplingParams

    eng = Engine(net, EngineConfig(-(-tokens // page) + 16, page, max_admit=1, max_running=1, cuda_graphs=graphs))
    g = torch.Generator().manual_seed(123)
    times = []
    for i in range(warmup + iters):
        ids = torch.randint(0, net.config.vocab_size, (tokens,), generator=g).tolist()
        req = eng.add(ids, SamplingParams(1))
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step()
        b.record()
        torch.cuda.synchronize()
        assert req.state == "done"
        if i >= warmup:
            times.append(a.elapsed_time(b))
    del eng
    torch.cuda.empty_cache()
    return sorted(times)[len(times) // 2]


def _measure(args, shape, rope, context, prefill_tokens, page, backend: str, sampler_cls) -> dict:
    import torch

    graphs = backend != "sdpa"
    net = _build_model({**shape, "num_hidden_layers": args.layers}, rope, backend)
    repeats = max(1, args.repeats)
    ms, host, spread, clocks = _decode_point(net, args.batch, context, args.steps, args.warmup, repeats, page, graphs, sampler_cls)
    points = {}
    for b in (1, 64):
        if backend == "sdpa" and b == 64:
            continue  # the per-request Python loop of that backend makes this point minutes long
        pms, _, _, _ = _decode_point(net, b, context, args.steps, args.warmup, repeats, page, graphs, sampler_cls)
        points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
    pre_ms = _prefill_point(net, prefill_tokens, page, warmup=2, iters=3, graphs=graphs)
    return {
        "impl": "reference",
        "reference_path": "FlashInferBackend + CUDA graphs (its default on a GPU)" if graphs else "SdpaBackend, cuda_graphs=False",
        "metric": f"decode tok/s (Llama-3.1-8B shape, batch {args.batch}, {context:,}-token context)",
        "value": round(args.batch * 1000.0 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform random token ids, random N(0, 0.02) weights",
        "config": {"model": "Llama-3.1-8B shape", "layers": args.layers, "layers_of_config": shape["num_hidden_layers"],
                   "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
                   "global_batch": args.batch, "seq_len": context, "max_context": shape["max_position_embeddings"], "page": page,
                   "parallelism": "single GPU", "cuda_graphs": graphs, "repeats": repeats,
                   "l2": "inputs larger than L2 (16 GB of weights per step)"},
        "e2e": {"value": round(args.batch / host, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 3 * 8 * args.batch, "d2h_bytes_per_step": 3 * 4 * args.batch},
        "ms_per_step_min_max": [round(spread[0], 4), round(spread[1], 4)],
        "prefill": {"value": round(prefill_tokens * 1000.0 / pre_ms, 1), "tokens": prefill_tokens, "ms": round(pre_ms, 3)},
        "points": points, "clocks": clocks, "torch": torch.__version__,
    }


def run(args, shape: dict, rope: tuple, context: int, prefill_tokens: int, page: int, sampler_cls) -> dict:
    missing = reference_present()
    if missing:
        return {"impl": "reference", "unavailable": missing}
    sys.path.insert(0, REF)
    try:
        import torch

        if not torch.cuda.is_available():
            return {"impl": "reference", "unavailable": "no CUDA device: the reference's engine path needs one"}
        return _measure(args, shape, rope, context, prefill_tokens, page, "auto", sampler_cls)
    except Exception:
        first = traceback.format_exc()
    tail = " | ".join(line.strip() for line in first.strip().splitlines()[-4:])[:600]
    try:
        import torch

        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        out = _measure(args, shape, rope, context, prefill_tokens, page, "sdpa", sampler_cls)
        out["default_path_error"] = tail
        return out
    except Exception:
        second = " | ".join(line.strip() for line in traceback.format_exc().strip().splitlines()[-3:])[:400]
        return {"impl": "reference", "unavailable": f"the reference's default path failed: {tail}; its sdpa path failed: {second}"}

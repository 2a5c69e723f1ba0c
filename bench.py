"""Decode and prefill throughput at the Llama-3.1-8B shape with random weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--repeats R] [--batch 8] [--layers 32] [--impl reference]

Prints ONE JSON line.  `value` is decoded tokens per second at the default batch (8 requests,
each with 1,024 tokens of context): after W warm-up steps, R repeats of K decode steps are timed
on the device with CUDA events and the median repeat is reported (`ms_per_step_min_max` gives the
spread).  `e2e` is the same workload through the Python entry point (`Engine.step`), with every
step's token ids going from pinned host memory to the device and the sampled tokens read back,
timed on the host clock.  `prefill` is one step of 2,048 prompt tokens; `roofline` sets the decode
step's bytes (every weight it uses once plus the cache of the live requests) against the measured
copy bandwidth.  `points` holds decode at batch 1 and 64 and two further workloads, each with its
time set against the roofline of its steps (a step's bound is the slower of its flops over the
tensor peak and its bytes over the copy peak): continuous batching of 64 requests at the
Llama-3.2-3B shape (prompts of 16 to 2,048 tokens, 256 new tokens each) and, at the Llama-3.2-1B
shape, 8 prompts of 8,192 tokens prefilled in portions of 512 beside 128 requests that decode
with temperature 1.0 and fixed seeds.  SM clocks are sampled during every point (`clocks` for the
headline point, `clocks_points` for the others).  The weights of every step are larger than L2,
so nothing is flushed between timed iterations.  Peaks come from MEASURED_PEAKS.json beside this
file when present.

`--impl reference` runs the same workloads on the unmodified reference engine (baseline/reference_arm.py).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# every size of the benchmark's third, fourth and fifth configuration
SHAPES = {
    "8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192),
    "3b": dict(vocab_size=128256, hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
               num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=4096,
               tie_word_embeddings=True),
    "1b": dict(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
               num_key_value_heads=8, head_dim=64, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=16384,
               tie_word_embeddings=True),
}
ROPES = {"8b": (8.0, 1.0, 4.0, 8192), "3b": (32.0, 1.0, 4.0, 8192), "1b": (32.0, 1.0, 4.0, 8192)}
SHAPE, ROPE = SHAPES["8b"], ROPES["8b"]
CONTEXT = 1024        # tokens each request holds when decoding is timed
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            p = json.load(open(path))
            out = dict(FALLBACK_PEAKS)

            def find(node, key):  # the key at the top level, or in a nested object
                if isinstance(node, dict):
                    if isinstance(node.get(key), (int, float)) and not isinstance(node.get(key), bool):
                        return float(node[key])
                    for v in node.values():
                        hit = find(v, key)
                        if hit is not None:
                            return hit
                return None

            found = {k: find(p, k) for k in out}
            if found["hbm_gbs"] is not None or found["bf16_tflops"] is not None:
                out.update({k: v for k, v in found.items() if v is not None and v > 0})
                return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.proc = None
        self.first = 0

    def mark(self) -> None:
        """The timed region begins: samples taken before now (nvidia-smi needs a moment to start, so it is started
        ahead of the warm-up) do not count, except the last one when no later sample exists."""
        self.first = len(self.rows)

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = self.rows[self.first:] or self.rows[-1:]
        sm = sorted(int(r[0]) for r in rows if len(r) >= 6 and r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


class Sizes:
    """Elements, bytes and flops of a shape, for setting times against the roofline."""

    def __init__(self, cfg: dict, layers: int) -> None:
        H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
        nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        self.layers, self.H, self.V, self.nq, self.d = layers, H, V, nq, d
        self.per_layer = (nq + 2 * nkv) * d * H + H * nq * d + 3 * I * H  # matrix elements of one layer
        self.head = V * H
        self.norms = (2 * layers + 1) * H
        self.kv_per_token = 2 * layers * nkv * d * 2                      # bytes, bf16

    def decode_bytes(self, batch: int, context: int) -> float:
        return 2 * (self.layers * self.per_layer + self.head) + 4 * self.norms + batch * self.H * 2 \
            + batch * context * self.kv_per_token

    def step_flops(self, tokens: int, sampled: int, pairs: int) -> float:
        """Products over `tokens` rows, the head over `sampled` rows, q k^T and p v over `pairs` query-key pairs."""
        return 2.0 * tokens * self.layers * self.per_layer + 2.0 * sampled * self.head + 4.0 * self.layers * self.nq * self.d * pairs

    def step_bytes(self, kv_positions: int, sampled: int) -> float:
        return 2.0 * (self.layers * self.per_layer + (self.head if sampled else 0)) + kv_positions * self.kv_per_token

    def step_bound_s(self, log_row: tuple, pk: dict) -> float:
        tokens, kv_positions, sampled, pairs = log_row
        return max(self.step_flops(tokens, sampled, pairs) / (pk["bf16_tflops_sustained"] * 1e12),
                   self.step_bytes(kv_positions, sampled) / (pk["hbm_gbs"] * 1e9))


def build_engine(shape: str, layers: int | None, max_running: int, num_blocks: int, **kw):
    import torch

    from nanospec_b200 import Engine, EngineConfig, LlamaConfig, random_model
    from nanospec_b200.config import Llama3RopeScaling

    sh = dict(SHAPES[shape])
    if layers:
        sh["num_hidden_layers"] = layers
    cfg = LlamaConfig(**sh, rope_scaling=Llama3RopeScaling(*ROPES[shape]))
    model = random_model(cfg, seed=0, device="cuda", dtype=torch.bfloat16)
    opts = dict(num_blocks=num_blocks, block_size=PAGE, max_running=max_running, max_admit=64, max_step_tokens=8192,
                prefill_chunk=PREFILL_TOKENS)
    opts.update(kw)
    return model, Engine(model, EngineConfig(**opts))


def prime(eng, batch: int, context: int, max_tokens: int, seed: int = 0):
    """Adds `batch` requests of `context` random tokens and runs steps until all of them decode."""
    import torch

    from nanospec_b200 import SamplingParams

    g = torch.Generator().manual_seed(seed)
    vocab = eng.model.vocab_size
    reqs = [eng.add(torch.randint(0, vocab, (context - 1,), generator=g).tolist(),
                    SamplingParams(max_tokens=max_tokens, ignore_eos=True)) for _ in range(batch)]
    while any(r.state == "waiting" or (r.state == "running" and r.pending > 1) for r in reqs):
        eng.step()
    return reqs


def median(xs: list[float]) -> float:
    xs = sorted(xs)
    return xs[len(xs) // 2]


def time_decode(eng, batch: int, steps: int, warmup: int, repeats: int) -> dict:
    """`repeats` x `steps` decode steps of `batch` requests after `warmup` steps.  Device time: every step is
    one graph launch with its own pair of events around copy-in, replay and copy-out; a repeat's figure is the
    mean over the launches made during it (steps may be launched one ahead of their predecessor's results, so a
    repeat's launches can differ from its calls by one).  Host time: the clock around the repeat's `step()` calls."""
    import torch

    from nanospec_b200.ops import lib

    sampler = ClockSampler()
    sampler.start()
    reqs = prime(eng, batch, CONTEXT, max_tokens=warmup + repeats * steps + 8)
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    bucket = eng.graphs.buckets[eng.graphs.bucket_size(batch)]
    launches0, replays0 = lib.launch_count(), eng.graphs.replays
    sampler.mark()
    dev_ms, host_s = [], []
    for _ in range(repeats):
        eng.graphs.timing = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.step()          # host ids -> pinned -> device, graph replay, sampled tokens back to the host
        torch.cuda.synchronize()
        host_s.append((time.perf_counter() - t0) / steps)
        launched = len(eng.graphs.timing)
        assert abs(launched - steps) <= 1, f"{launched} graph launches in {steps} timed steps"
        dev_ms.append(sum(s.elapsed_time(e) for s, e in eng.graphs.timing) / launched)
    clocks = sampler.stop()
    eng.graphs.timing = None
    launches = lib.launch_count() - launches0 + (eng.graphs.replays - replays0) * bucket.kernels
    h2d = eng.runner.h2d_bytes_last
    for r in reqs:
        if r.state == "running":
            eng.sched.finish(r)
    return {"ms": median(dev_ms), "ms_min": min(dev_ms), "ms_max": max(dev_ms), "host_s": median(host_s), "clocks": clocks,
            "launches": launches, "h2d": h2d, "d2h": 3 * 4 * batch}


def time_prefill(eng, warmup: int, iters: int) -> tuple[float, dict]:
    import torch

    from nanospec_b200 import SamplingParams

    g = torch.Generator().manual_seed(123)
    times = []
    sampler = ClockSampler()
    sampler.start()
    for i in range(warmup + iters):
        if i == warmup:
            sampler.mark()
        ids = torch.randint(0, eng.model.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
        req = eng.add(ids, SamplingParams(max_tokens=1, ignore_eos=True))
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step()
        b.record()
        torch.cuda.synchronize()
        assert req.state == "done"
        if i >= warmup:
            times.append(a.elapsed_time(b))
    return median(times), sampler.stop()


def _workload_record(eng, sizes: Sizes, pk: dict, seconds: float, out_tokens: int, all_tokens: int, live: int, clocks: dict) -> dict:
    bound = sum(sizes.step_bound_s(row, pk) for row in eng.step_log)
    return {"out_tok_s": round(out_tokens / seconds, 1), "total_tok_s": round(all_tokens / seconds, 1),
            "tpot_ms": round(1000.0 * seconds / (out_tokens / live), 3), "seconds": round(seconds, 4), "steps": len(eng.step_log),
            "roofline_s": round(bound, 4), "frac": round(bound / seconds, 4), "sm_mhz": clocks.get("sm_mhz"),
            "reasons": clocks.get("reasons")}


def workload_continuous_batching(pk: dict, runs: int) -> dict:
    """Llama-3.2-3B shape: 64 requests with prompts of 16 to 2,048 seeded random tokens and 256 new tokens each,
    all admitted at once, continuous batching until the last one ends.  The reference's definitions
    (bench/run.py:43-44, bench/table.py:19 there): tok_s = output tokens / seconds, tpot_ms = 1000 * seconds /
    (output tokens / batch), the median over the runs; the first run also loads the library's kernels for these
    shapes and does not count."""
    import torch

    from nanospec_b200 import SamplingParams

    n_req, new = 64, 256
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16, 2048 + 1, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, SHAPES["3b"]["vocab_size"], (n,), generator=g).tolist() for n in lens]
    pages = sum(-(-(n + new) // PAGE) + 1 for n in lens) + 16
    model, eng = build_engine("3b", None, n_req, pages)
    sizes = Sizes(SHAPES["3b"], SHAPES["3b"]["num_hidden_layers"])
    recs = []
    for run in range(runs + 1):
        eng.step_log = []
        sampler = ClockSampler()
        sampler.start()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = eng.generate(prompts, SamplingParams(max_tokens=new, ignore_eos=True))
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        n_out = sum(len(o) for o in outs)
        recs.append(_workload_record(eng, sizes, pk, dt, n_out, n_out + sum(lens), n_req, sampler.stop()))
    recs = sorted(recs[1:], key=lambda r: r["seconds"])
    rec = recs[len(recs) // 2]
    rec.update(requests=n_req, prompt_tokens=sum(lens), new_tokens_each=new, runs=runs, context=4096)
    del eng, model
    torch.cuda.empty_cache()
    return rec


def workload_mixed(pk: dict, runs: int) -> dict:
    """Llama-3.2-1B shape, contexts of up to 16,384: 128 requests decode (temperature 1.0, fixed seeds) while 8
    prompts of 8,192 tokens are prefilled in portions of 512.  Timed from the step that admits the prompts to the
    step that ends the last of them; the decoders run throughout."""
    import torch

    from nanospec_b200 import SamplingParams

    n_dec, n_long, long_len, portion = 128, 8, 8192, 512
    vocab = SHAPES["1b"]["vocab_size"]
    g = torch.Generator().manual_seed(0)
    dec = [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in torch.randint(32, 512, (n_dec,), generator=g)]
    longs = [torch.randint(0, vocab, (long_len,), generator=g).tolist() for _ in range(n_long)]
    budget = (runs + 1) * (long_len // portion + 8) + 32   # the decoders outlive every run's prompts
    pages = sum(-(-(len(p) + budget) // PAGE) + 1 for p in dec) + n_long * (long_len // PAGE + 8) + 16
    model, eng = build_engine("1b", None, n_dec + n_long, pages, prefill_chunk=portion)
    sizes = Sizes(SHAPES["1b"], SHAPES["1b"]["num_hidden_layers"])
    reqs = [eng.add(p, SamplingParams(max_tokens=budget, temperature=1.0, seed=7 + i, ignore_eos=True)) for i, p in enumerate(dec)]
    while any(r.state == "waiting" or (r.state == "running" and r.pending > 1) for r in reqs):
        eng.step()
    recs = []
    for run in range(runs + 1):
        lreqs = [eng.add(p, SamplingParams(max_tokens=2, temperature=1.0, seed=99 + i, ignore_eos=True)) for i, p in enumerate(longs)]
        eng.step_log = []
        sampler = ClockSampler()
        sampler.start()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while any(r.state != "done" for r in lreqs):
            eng.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        steps = len(eng.step_log)
        n_out = steps * n_dec + 2 * n_long
        rec = _workload_record(eng, sizes, pk, dt, n_out, n_out + n_long * long_len, n_dec, sampler.stop())
        rec["prefill_tok_s"] = round(n_long * long_len / dt, 1)
        rec["ms_per_step"] = round(1000.0 * dt / steps, 3)
        recs.append(rec)
    assert all(r.state == "running" for r in reqs)
    recs = sorted(recs[1:], key=lambda r: r["seconds"])
    rec = recs[len(recs) // 2]
    rec.update(decoding_requests=n_dec, long_prompts=n_long, prompt_tokens_each=long_len, portion=portion, temperature=1.0,
               runs=runs, context=16384)
    del eng, model
    torch.cuda.empty_cache()
    return rec


def run_ours(args) -> dict:
    import torch

    pk, pk_src = peaks()
    layers = args.layers
    sizes = Sizes(SHAPE, layers)
    pages_per_req = -(-(CONTEXT + args.repeats * args.steps + args.warmup + 64) // PAGE)
    num_blocks = max(64 * pages_per_req, -(-PREFILL_TOKENS // PAGE) + 8) + 8
    model, eng = build_engine("8b", layers, 64, num_blocks)
    torch.cuda.synchronize()

    head = time_decode(eng, args.batch, args.steps, args.warmup, args.repeats)
    dev_ms = head["ms"]
    value = args.batch * 1000.0 / dev_ms
    e2e = args.batch / head["host_s"]

    points, clocks_points = {}, {}
    for b in (1, 64):
        pt = time_decode(eng, b, args.steps, args.warmup, args.repeats)
        points[f"decode_b{b}"] = round(b * 1000.0 / pt["ms"], 1)
        points[f"decode_b{b}_frac"] = round(sizes.decode_bytes(b, CONTEXT) / (pt["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        clocks_points[f"decode_b{b}"] = {"sm_mhz": pt["clocks"].get("sm_mhz"), "reasons": pt["clocks"].get("reasons"),
                                         "ms": round(pt["ms"], 4), "ms_min_max": [round(pt["ms_min"], 4), round(pt["ms_max"], 4)]}
    pre_ms, pre_clocks = time_prefill(eng, warmup=3, iters=5)
    clocks_points["prefill"] = {"sm_mhz": pre_clocks.get("sm_mhz"), "reasons": pre_clocks.get("reasons")}
    prefill_flops = sizes.step_flops(PREFILL_TOKENS, 1, PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2)
    del eng, model
    torch.cuda.empty_cache()

    workloads = {}
    if not args.no_workloads and layers == SHAPE["num_hidden_layers"]:
        workloads["continuous_batching_3b"] = workload_continuous_batching(pk, runs=3)
        workloads["mixed_1b"] = workload_mixed(pk, runs=3)
        for name, short in (("continuous_batching_3b", "cb3b"), ("mixed_1b", "mixed1b")):
            for key in ("out_tok_s", "total_tok_s", "tpot_ms", "frac"):
                points[f"{short}_{key}"] = workloads[name][key]

    achieved = sizes.decode_bytes(args.batch, CONTEXT) / (dev_ms * 1e-3) / 1e9
    mhz = head["clocks"].get("sm_mhz")
    return {
        "metric": "decode tok/s (Llama-3.1-8B shape, batch 8, 1,024-token context)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform random token ids, random N(0, 0.02) weights",
        "config": {"model": "Llama-3.1-8B shape", "layers": layers, "layers_of_config": SHAPE["num_hidden_layers"],
                   "hidden": SHAPE["hidden_size"], "heads": SHAPE["num_attention_heads"],
                   "kv_heads": SHAPE["num_key_value_heads"], "head_dim": SHAPE["head_dim"],
                   "intermediate": SHAPE["intermediate_size"], "vocab": SHAPE["vocab_size"], "global_batch": args.batch,
                   "seq_len": CONTEXT, "max_context": SHAPE["max_position_embeddings"], "page": PAGE,
                   "parallelism": "single GPU", "cuda_graphs": True, "repeats": args.repeats,
                   "l2": "inputs larger than L2 (16 GB of weights per step)",
                   "peaks": pk_src},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": head["h2d"], "d2h_bytes_per_step": head["d2h"]},
        "gpu_launches": head["launches"],
        "ms_per_step_min_max": [round(head["ms_min"], 4), round(head["ms_max"], 4)],
        "ms_x_sm_mhz": round(dev_ms * mhz, 1) if mhz else None,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(prefill_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_of_sustained": round(prefill_flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "workloads": workloads,
        # the one number the reference publishes for this architecture: 137 tok/s at batch 1 on an H100
        # (its README.md:76); the headline metric here (batch 8) has no published counterpart
        "vs_published_b1_h100": round(points["decode_b1"] / 137.0, 2),
        "clocks": head["clocks"],
        "clocks_points": clocks_points,
    }


def run_reference(args) -> dict:
    from baseline import reference_arm

    return reference_arm.run(args, SHAPE, ROPE, CONTEXT, PREFILL_TOKENS, PAGE, ClockSampler)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5, help="the timed steps are run this many times; the median repeat is reported")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=SHAPE["num_hidden_layers"])
    ap.add_argument("--no-workloads", action="store_true", help="leave out the 3B continuous-batching and 1B mixed workloads")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    args.repeats = max(1, args.repeats)
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())

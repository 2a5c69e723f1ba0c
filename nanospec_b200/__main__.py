"""Command line: `python -m nanospec_b200 <command> ...`.

    generate        run prompts of token ids through the engine, print one JSON line per prompt
    bench           the reference's harness in this engine's terms (python -m bench.run nanospec
                    --config nospec --bs 1 8 32 --max-tokens 256 --runs 3 there, bench/run.py:162-177):
                    one JSON line per (batch size, run) with tok_s and tpot_ms
    random-weights  write a model folder with seeded random weights from sizes or a config.json
    profile         one decode or prefill step at a named shape, bracketed for a profiler
    replay          trace replay (the same program as bin/trace_run)
    table           fold the JSON lines of `bench` into a table, the median over the runs of each batch size
                    (python -m bench.table there, bench/table.py:11-23)

The model folder comes from --model or the NANOSPEC_MODEL environment variable, as in the
reference (bench/run.py:24).  Token ids go in and come out; there is no tokenizer inside.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _model_arg(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", default=os.environ.get("NANOSPEC_MODEL"), help="model folder (or $NANOSPEC_MODEL)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")


def _engine_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--num-blocks", type=int, default=None, help="cache pages (default: sized for the workload)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-running", type=int, default=None)
    ap.add_argument("--max-admit", type=int, default=32)
    ap.add_argument("--max-step-tokens", type=int, default=8192)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--admission", choices=["reserve", "optimistic"], default="reserve")
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--no-lookahead", action="store_true", help="never launch a step before the one before it has been read")


def _load(args):
    import torch

    from .weights import load_model

    if not args.model:
        sys.exit("no model folder: give --model or set NANOSPEC_MODEL")
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    return load_model(args.model, device="cuda", dtype=dtype)


def _engine(model, args, num_blocks: int):
    from .config import EngineConfig
    from .engine import Engine

    return Engine(model, EngineConfig(
        num_blocks=args.num_blocks or num_blocks, block_size=args.block_size, max_admit=args.max_admit,
        max_running=args.max_running, cuda_graphs=not args.no_cuda_graphs, max_step_tokens=args.max_step_tokens,
        prefill_chunk=args.prefill_chunk, admission=args.admission, lookahead=not args.no_lookahead))


def cmd_generate(args) -> int:
    import torch

    from .engine import SamplingParams

    model = _load(args)
    prompts: list[list[int]] = []
    for p in args.prompt_ids or []:
        prompts.append([int(t) for t in p.replace(",", " ").split()])
    if args.prompt_lens:
        g = torch.Generator().manual_seed(args.seed or 0)
        for n in args.prompt_lens:
            prompts.append(torch.randint(0, model.vocab_size, (n,), generator=g).tolist())
    if not prompts:
        sys.exit("no prompts: give --prompt-ids '1 2 3' (repeatable) or --prompt-lens N ...")
    need = sum(-(-(len(p) + args.max_tokens) // args.block_size) for p in prompts) + 1
    engine = _engine(model, args, need)
    params = [SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                             seed=None if args.seed is None else args.seed + i, ignore_eos=args.ignore_eos)
              for i in range(len(prompts))]
    t0 = time.perf_counter()
    outs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for i, (p, o) in enumerate(zip(prompts, outs)):
        print(json.dumps({"request": i, "prompt_len": len(p), "output_ids": o}), flush=True)
    n_out = sum(len(o) for o in outs)
    print(json.dumps({"requests": len(prompts), "out_tokens": n_out, "seconds": round(dt, 4),
                      "tok_s": round(n_out / dt, 1), "steps": engine.steps}), flush=True)
    return 0


def cmd_bench(args) -> int:
    import torch

    from .engine import SamplingParams

    model = _load(args)
    g = torch.Generator().manual_seed(0)
    base = [torch.randint(0, model.vocab_size, (args.prompt_len,), generator=g).tolist() for _ in range(args.prompts)]
    prompts = [p for p in base for _ in range(args.n_samples)]
    # one engine per (batch size, run), as the reference's harness builds them (bench/run.py:75-91): `bs` live requests at
    # most and at most 8 admissions per step; the clock covers adding every prompt and stepping until none is left
    for bs, run in ((bs, run) for bs in args.bs for run in range(args.runs)):
        args.max_running, args.max_admit = bs, min(bs, 8)
        pages_each = -(-(args.prompt_len + args.max_tokens) // args.block_size) + 1
        engine = _engine(model, args, bs * pages_each)
        plist = [SamplingParams(args.max_tokens, temperature=args.temperature, seed=i, ignore_eos=True) for i in range(len(prompts))]
        torch.cuda.synchronize()
        started = time.perf_counter()
        outs = engine.generate(prompts, plist)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - started
        n_out = sum(len(o) for o in outs)
        print(json.dumps({
            "engine": "nanospec_b200", "config": "nospec", "bs": bs, "prompts": len(prompts), "out_tokens": n_out,
            "tok_s": round(n_out / seconds, 1), "tpot_ms": round(1000 * seconds / (n_out / bs), 2), "run": run,
            "temperature": args.temperature, "gpu": torch.cuda.get_device_name(0), "dtype": args.dtype,
            "steps": engine.steps, "data": "seeded uniform random token ids"}), flush=True)
        del engine
        torch.cuda.empty_cache()
    return 0


def fold_bench_lines(lines) -> str:
    """The lines that `bench` printed (anything that does not open with a brace is skipped), folded into a
    markdown table: one row per (engine, config, batch size) with the medians of its runs."""
    import statistics

    groups: dict[tuple, list[dict]] = {}
    for line in lines:
        line = line.strip()
        if line.startswith("{"):
            row = json.loads(line)
            groups.setdefault((row.get("engine", "?"), row.get("config", "?"), row.get("bs", 0)), []).append(row)
    out = ["| engine | config | bs | out tok/s | TPOT ms | runs | dtype | gpu |", "|---|---|---|---|---|---|---|---|"]
    for (engine, config, bs), rows in sorted(groups.items()):
        def median(key: str):
            vals = [r[key] for r in rows if r.get(key) is not None]
            return round(statistics.median(vals), 2) if vals else "-"
        out.append(f"| {engine} | {config} | {bs} | {median('tok_s')} | {median('tpot_ms')} | {len(rows)} | "
                   f"{rows[0].get('dtype', '-')} | {rows[0].get('gpu', '-')} |")
    return "\n".join(out)


def cmd_table(args) -> int:
    lines: list[str] = []
    for path in args.files or ["-"]:
        if path == "-":
            lines.extend(sys.stdin)
        else:
            with open(path) as f:
                lines.extend(f)
    print(fold_bench_lines(lines))
    return 0


def cmd_profile(args) -> int:
    """Decode steps, or the prefill of one batch of prompts, at a named shape with random weights,
    bracketed by cudaProfilerStart/Stop so that a profiler started with --profile-from-start off sees
    only them.  Prints the median step time, tokens per second and (decode) the bytes a step has to
    read over its time."""
    import torch

    from .config import Llama3RopeScaling, LlamaConfig
    from .engine import SamplingParams
    from .weights import random_model

    shapes = {
        "8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_attention_heads=32,
                   num_key_value_heads=8, head_dim=128, layers=32, factor=8.0),
        "3b": dict(vocab_size=128256, hidden_size=3072, intermediate_size=8192, num_attention_heads=24,
                   num_key_value_heads=8, head_dim=128, layers=28, factor=32.0, tie_word_embeddings=True),
        "1b": dict(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_attention_heads=32,
                   num_key_value_heads=8, head_dim=64, layers=16, factor=32.0, tie_word_embeddings=True),
    }
    sh = dict(shapes[args.shape])
    layers = args.layers or sh.pop("layers")
    sh.pop("layers", None)
    factor = sh.pop("factor")
    cfg = LlamaConfig(**sh, num_hidden_layers=layers, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=max(8192, args.context + 512), rope_scaling=Llama3RopeScaling(factor, 1.0, 4.0, 8192))
    model = random_model(cfg, seed=0, device="cuda", dtype=torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    if args.what in ("batch", "mixed", "queue"):
        return _profile_workload(args, cfg, model)
    args.max_running = max(args.batch, 1)
    args.max_admit = 64
    pages = (args.batch + (1 if args.what == "prefill" else 0)) * (-(-(args.context + 256 + args.steps) // args.block_size) + 1) + 8
    engine = _engine(model, args, pages)
    g = torch.Generator().manual_seed(0)
    n_prompt = args.context - 1 if args.what == "decode" else args.context
    reqs = [engine.add(torch.randint(0, cfg.vocab_size, (n_prompt,), generator=g).tolist(),
                       SamplingParams(max_tokens=256 + args.steps if args.what == "decode" else 1, ignore_eos=True))
            for _ in range(args.batch)]
    if args.what == "decode":
        while any(r.state == "waiting" or (r.state == "running" and r.pending > 1) for r in reqs):
            engine.step()
        for _ in range(3):
            engine.step()
    else:
        warm = engine.add(torch.randint(0, cfg.vocab_size, (n_prompt,), generator=g).tolist(),
                          SamplingParams(max_tokens=1, ignore_eos=True))
        engine.sched.waiting.remove(warm)
        engine.sched.waiting.appendleft(warm)
        engine.sched.max_admit = 1
        while warm.state != "done":   # a prompt longer than a portion takes several steps
            engine.step()
        engine.sched.max_admit = 64
    torch.cuda.synchronize()
    times = []
    torch.cuda.profiler.start()
    if args.what == "decode":
        for _ in range(args.steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            engine.step()
            b.record()
            times.append((a, b))
    else:
        while any(r.state != "done" for r in reqs):   # every portion of every prompt
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            engine.step()
            b.record()
            times.append((a, b))
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ms = sorted(a.elapsed_time(b) for a, b in times)
    out = {"what": args.what, "shape": args.shape, "layers": layers, "batch": args.batch, "context": args.context,
           "graphs": not args.no_cuda_graphs, "steps": len(ms), "step_ms": round(ms[len(ms) // 2], 3)}
    if args.what == "decode":
        per_layer = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim * cfg.hidden_size \
            + cfg.hidden_size * cfg.num_attention_heads * cfg.head_dim + 3 * cfg.intermediate_size * cfg.hidden_size
        elt = 2 if args.dtype == "bfloat16" else 4
        step_bytes = elt * (layers * per_layer + cfg.vocab_size * cfg.hidden_size) \
            + args.batch * args.context * 2 * layers * cfg.num_key_value_heads * cfg.head_dim * elt
        out["tokens_per_s"] = round(args.batch * 1000.0 / out["step_ms"], 1)
        out["gb_per_s"] = round(step_bytes / (out["step_ms"] * 1e-3) / 1e9, 1)
    else:
        out["total_ms"] = round(sum(ms), 3)
        out["tokens_per_s"] = round(args.batch * args.context * 1000.0 / sum(ms), 1)
    print(json.dumps(out), flush=True)
    return 0


def _profile_workload(args, cfg, model) -> int:
    """`queue`: --requests requests through --batch live slots, so that somebody always waits.
    `batch`: continuous batching of --batch requests with prompt lengths uniform in [--prompt-min, --context] and
    --new-tokens new tokens each.  `mixed`: --long prompts of --context tokens prefilled in portions of
    --prefill-chunk beside --batch requests that decode (temperature 1.0, fixed seeds)."""
    import time

    import torch

    from .engine import SamplingParams

    g = torch.Generator().manual_seed(0)
    bs = args.block_size
    if args.what == "queue":
        n_req = args.requests or 3 * args.batch
        lens = torch.randint(args.prompt_min, args.context + 1, (n_req,), generator=g).tolist()
        news = torch.randint(max(1, args.new_tokens // 4), args.new_tokens + 1, (n_req,), generator=g).tolist()
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
        args.max_running, args.max_admit = args.batch, 64
        runs = []
        for _ in range(2):  # the second run is the one that counts: the first also warms the library's kernels up
            engine = _engine(model, args, args.batch * (-(-(args.context + args.new_tokens) // bs) + 1) + 16)
            for p, n in zip(prompts, news):
                engine.add(p, SamplingParams(max_tokens=n, ignore_eos=True))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            while engine.sched.has_work:
                engine.step()
            torch.cuda.synchronize()
            runs.append(time.perf_counter() - t0)
        dt = runs[-1]
        print(json.dumps({"what": "queue", "shape": args.shape, "requests": n_req, "live": args.batch, "prompt_tokens": sum(lens),
                          "new_tokens": sum(news), "seconds": round(dt, 3), "steps": engine.steps, "launched_ahead": engine.launched_ahead,
                          "new_tokens_per_s": round(sum(news) / dt, 1)}), flush=True)
        return 0
    if args.what == "batch":
        lens = torch.randint(args.prompt_min, args.context + 1, (args.batch,), generator=g).tolist()
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
        args.max_running, args.max_admit = args.batch, 64
        runs = []
        for _ in range(2):  # the second run is the one that counts: the first also loads the library's kernels for these shapes
            engine = _engine(model, args, sum(-(-(n + args.new_tokens) // bs) + 1 for n in lens) + 16)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = engine.generate(prompts, SamplingParams(max_tokens=args.new_tokens, ignore_eos=True))
            torch.cuda.synchronize()
            runs.append(time.perf_counter() - t0)
        dt = runs[-1]
        new = sum(len(o) for o in outs)
        print(json.dumps({"what": "batch", "shape": args.shape, "requests": args.batch, "prompt_tokens": sum(lens), "new_tokens": new,
                          "seconds": round(dt, 3), "first_run_seconds": round(runs[0], 3), "steps": engine.steps,
                          "new_tokens_per_s": round(new / dt, 1), "all_tokens_per_s": round((sum(lens) + new) / dt, 1)}), flush=True)
        return 0
    dec = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist()
           for n in torch.randint(32, 512, (args.batch,), generator=g)]
    longs = [torch.randint(0, cfg.vocab_size, (args.context,), generator=g).tolist() for _ in range(args.long)]
    args.max_running, args.max_admit = args.batch + args.long, 64
    pages = sum(-(-(len(p) + 4 * args.context // args.prefill_chunk + 64) // bs) + 1 for p in dec) + args.long * (args.context // bs + 8) + 16
    engine = _engine(model, args, pages)
    budget = 4 * args.context // args.prefill_chunk + 32   # the decoders outlive the prompts
    reqs = [engine.add(p, SamplingParams(max_tokens=budget, temperature=1.0, seed=7 + i, ignore_eos=True)) for i, p in enumerate(dec)]
    while any(r.state == "waiting" or (r.state == "running" and r.pending > 1) for r in reqs):
        engine.step()
    lreqs = [engine.add(p, SamplingParams(max_tokens=2, temperature=1.0, seed=99 + i, ignore_eos=True)) for i, p in enumerate(longs)]
    torch.cuda.synchronize()
    t0, s0 = time.perf_counter(), engine.steps
    h0 = (engine.host_compose_s, engine.host_launch_s)
    while any(r.state != "done" for r in lreqs):
        if args.sync_steps:
            torch.cuda.synchronize()  # an empty launch queue: the host timers then hold the host's own work only
        engine.step()
    torch.cuda.synchronize()
    dt, steps = time.perf_counter() - t0, engine.steps - s0
    host = (engine.host_compose_s - h0[0], engine.host_launch_s - h0[1])
    print(json.dumps({"what": "mixed", "shape": args.shape, "decoding_requests": args.batch, "long_prompts": args.long,
                      "prompt_tokens_each": args.context, "portion": args.prefill_chunk, "seconds": round(dt, 3), "steps": steps,
                      "ms_per_step": round(1000 * dt / steps, 3), "prefill_tokens_per_s": round(args.long * args.context / dt, 1),
                      "decoded_meanwhile": steps * args.batch, "launched_ahead": engine.launched_ahead,
                      "host_compose_ms_per_step": round(1000 * host[0] / steps, 3),
                      "host_launch_ms_per_step": round(1000 * host[1] / steps, 3)}), flush=True)
    return 0


def cmd_random_weights(args) -> int:
    from .config import Llama3RopeScaling, LlamaConfig
    from .weights import write_random_model

    if args.config:
        cfg = json.loads(open(args.config).read())
    else:
        scaling = None
        if args.rope_scaling:
            f, lo, hi, orig = args.rope_scaling
            scaling = Llama3RopeScaling(float(f), float(lo), float(hi), int(orig))
        cfg = LlamaConfig(
            vocab_size=args.vocab_size, hidden_size=args.hidden_size, intermediate_size=args.intermediate_size,
            num_hidden_layers=args.num_hidden_layers, num_attention_heads=args.num_attention_heads,
            num_key_value_heads=args.num_key_value_heads or args.num_attention_heads,
            head_dim=args.head_dim or args.hidden_size // args.num_attention_heads, rms_norm_eps=args.rms_norm_eps,
            rope_theta=args.rope_theta, max_position_embeddings=args.max_position_embeddings, rope_scaling=scaling,
            tie_word_embeddings=args.tie_word_embeddings)
    print(write_random_model(args.out, cfg, seed=args.seed))
    return 0


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m nanospec_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate from prompts of token ids")
    _model_arg(g), _engine_args(g)
    g.add_argument("--prompt-ids", action="append", help="one prompt as ids separated by spaces or commas (repeatable)")
    g.add_argument("--prompt-lens", type=int, nargs="+", help="seeded random prompts of these lengths")
    g.add_argument("--max-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--ignore-eos", action="store_true")
    g.set_defaults(fn=cmd_generate)

    b = sub.add_parser("bench", help="throughput over batch sizes, one JSON line per run")
    _model_arg(b), _engine_args(b)
    b.add_argument("--bs", type=int, nargs="+", default=[1, 8, 32])
    b.add_argument("--max-tokens", type=int, default=256)
    b.add_argument("--runs", type=int, default=3)
    b.add_argument("--temperature", type=float, default=0.0)
    b.add_argument("--n-samples", type=int, default=1, help="repeat every prompt this many times")
    b.add_argument("--prompts", type=int, default=80, help="number of distinct prompts")
    b.add_argument("--prompt-len", type=int, default=64)
    b.set_defaults(fn=cmd_bench)

    pr = sub.add_parser("profile", help="one step at a named shape between cudaProfilerStart/Stop (for ncu)")
    _engine_args(pr)
    pr.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    pr.add_argument("--shape", choices=["8b", "3b", "1b"], default="8b")
    pr.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (smaller captures)")
    pr.add_argument("--batch", type=int, default=8)
    pr.add_argument("--context", type=int, default=1024)
    pr.add_argument("--what", choices=["decode", "prefill", "batch", "mixed", "queue"], default="decode",
                    help="decode steps; the prefill of --batch prompts; batch: continuous batching of --batch requests; "
                         "mixed: --long prompts prefilled in portions beside --batch decoding requests")
    pr.add_argument("--prompt-min", type=int, default=16, help="batch: shortest prompt (the longest is --context)")
    pr.add_argument("--new-tokens", type=int, default=256, help="batch: new tokens per request")
    pr.add_argument("--long", type=int, default=8, help="mixed: number of long prompts")
    pr.add_argument("--requests", type=int, default=None,
                    help="queue: requests in all (default 3 x --batch), through --batch live slots; prompts of --prompt-min to "
                         "--context tokens, --new-tokens / 4 to --new-tokens new ones")
    pr.add_argument("--steps", type=int, default=1, help="decode steps to time (the median is printed)")
    pr.add_argument("--sync-steps", action="store_true",
                    help="mixed: wait for the GPU before every step, so that host_compose_ms and host_launch_ms hold the "
                         "host's own work and no waiting for room in the launch queue (use with --no-lookahead)")
    pr.set_defaults(fn=cmd_profile)

    r = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--config", help="a config.json to take every size from")
    r.add_argument("--vocab-size", type=int, default=256)
    r.add_argument("--hidden-size", type=int, default=64)
    r.add_argument("--intermediate-size", type=int, default=128)
    r.add_argument("--num-hidden-layers", type=int, default=2)
    r.add_argument("--num-attention-heads", type=int, default=8)
    r.add_argument("--num-key-value-heads", type=int, default=None)
    r.add_argument("--head-dim", type=int, default=None)
    r.add_argument("--rms-norm-eps", type=float, default=1e-5)
    r.add_argument("--rope-theta", type=float, default=10000.0)
    r.add_argument("--rope-scaling", nargs=4, metavar=("FACTOR", "LOW", "HIGH", "ORIGINAL_MAX_POS"),
                   help="llama3 frequency rescale")
    r.add_argument("--max-position-embeddings", type=int, default=256)
    r.add_argument("--tie-word-embeddings", action="store_true")
    r.set_defaults(fn=cmd_random_weights)

    tb = sub.add_parser("table", help="fold bench JSON lines (files, or standard input) into a table of medians")
    tb.add_argument("files", nargs="*", help="files of JSON lines; none or - reads standard input")
    tb.set_defaults(fn=cmd_table)

    p = sub.add_parser("replay", help="trace replay; same options as bin/trace_run", add_help=False)
    p.set_defaults(fn=None)

    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main

        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())

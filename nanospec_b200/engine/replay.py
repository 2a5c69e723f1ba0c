"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the same
`ModelRunner` (model, step function, cache manager, kernels) that generation uses.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch.  `want` lists the places among the entry's tokens
whose logits are written; `end` lists requests that are finished after the step and whose
pages go back to the pool.  For a step with wanted places the program writes
`<out>/<step>.f32`: little-endian float32 [wanted, vocab] in the order of the entries and of
their `want` lists.  After every step it prints `done <step>` and flushes.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--max-requests", type=int, default=8, help="most requests live at a time")
    args = ap.parse_args(argv)
    if 64 % args.block_size:
        ap.error("--block-size must divide 64")

    from .. import ops
    from ..ops import lib
    from ..weights import load_model
    from .step import ModelRunner, StepEntry

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 2
    lib.load()  # compiles the kernels on the first call, printing progress to stderr
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    model = load_model(args.model, device="cuda", dtype=dtype)
    num_blocks = max(1, -(-args.max_tokens // args.block_size))
    runner = ModelRunner(model, num_blocks=num_blocks, block_size=args.block_size, max_requests=args.max_requests)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    ids: dict[str, int] = {}
    next_id = 0
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            name = str(e["id"])
            if name not in ids:
                ids[name] = next_id
                next_id += 1
                runner.begin(ids[name])
            entries.append(StepEntry(ids[name], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                host = logits.to("cpu", torch.float32).contiguous()
                ops.check_kernel_errors()
                (out_dir / f"{step}.f32").write_bytes(host.numpy().astype("<f4", copy=False).tobytes())
        for name in rec.get("end", []):
            name = str(name)
            if name in ids:
                runner.end(ids.pop(name))
        print(f"done {step}", flush=True)
    torch.cuda.synchronize()
    runner.manager.check()
    return 0


if __name__ == "__main__":
    sys.exit(main())

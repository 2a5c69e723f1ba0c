"""Helpers for the replay tests: run bin/trace_run as a user would (a subprocess fed JSON
lines), build traces that cut the same sequences in different ways, and collect the logits
of every (request, position)."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"


def run_trace(folder, dtype: str, steps: list[dict], max_tokens: int, out_dir, block_size: int = 16,
              vocab: int | None = None, timeout: float = 600.0) -> dict[int, np.ndarray]:
    """Feeds `steps` to bin/trace_run one at a time, waiting for each `done <step>` line
    before sending the next, and returns {step: float32 [wanted, vocab]}."""
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(TRACE_RUN), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(max_tokens), "--block-size", str(block_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    try:
        for rec in steps:
            proc.stdin.write(json.dumps(rec) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == f"done {rec['step']}", f"trace_run answered {line!r} to step {rec['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    results = {}
    for rec in steps:
        n_want = sum(len(e.get("want", [])) for e in rec["entries"])
        path = out_dir / f"{rec['step']}.f32"
        if n_want:
            data = np.fromfile(path, dtype="<f4")
            results[rec["step"]] = data.reshape(n_want, -1)
            if vocab is not None:
                assert results[rec["step"]].shape[1] == vocab
        else:
            assert not path.exists()
    return results


def collect(steps: list[dict], results: dict[int, np.ndarray], seqs: dict[str, list[int]]) -> dict[str, np.ndarray]:
    """{request: float32 [len, vocab]} from the per-step outputs; every position must have
    been wanted exactly once."""
    vocab = next(iter(results.values())).shape[1]
    out = {name: np.full((len(ids), vocab), np.nan, dtype=np.float32) for name, ids in seqs.items()}
    cursor = {name: 0 for name in seqs}
    for rec in steps:
        row = 0
        for e in rec["entries"]:
            name, start = e["id"], cursor[e["id"]]
            assert e["tokens"] == seqs[name][start:start + len(e["tokens"])]
            for w in e.get("want", []):
                assert np.isnan(out[name][start + w, 0]), "a position was wanted twice"
                out[name][start + w] = results[rec["step"]][row]
                row += 1
            cursor[name] = start + len(e["tokens"])
    for name, arr in out.items():
        assert not np.isnan(arr).any(), f"request {name}: some positions were never wanted"
    return out


def _entry(name, seq, start, n):
    return {"id": name, "tokens": seq[start:start + n], "want": list(range(n))}


def trace_whole(seqs: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one step each."""
    return [{"step": i, "entries": [_entry(name, seq, 0, len(seq))], "end": [name]}
            for i, (name, seq) in enumerate(seqs.items())]


def trace_tail(seqs: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps, s = [], 0
    for name, seq in seqs.items():
        head = max(1, len(seq) - tail)
        steps.append({"step": s, "entries": [_entry(name, seq, 0, head)], "end": []})
        s += 1
        for p in range(head, len(seq)):
            steps.append({"step": s, "entries": [_entry(name, seq, p, 1)], "end": [name] if p == len(seq) - 1 else []})
            s += 1
        if head == len(seq):
            steps[-1]["end"] = [name]
    return steps


def trace_portions(seqs: dict[str, list[int]], sizes=(7, 2, 24, 5, 1, 16, 2, 33, 3, 64, 2, 9)) -> list[dict]:
    """Each request alone, in portions of changing size (down to two tokens and one)."""
    steps, s, k = [], 0, 0
    for name, seq in seqs.items():
        p = 0
        while p < len(seq):
            n = min(sizes[k % len(sizes)], len(seq) - p)
            k += 1
            steps.append({"step": s, "entries": [_entry(name, seq, p, n)], "end": [name] if p + n == len(seq) else []})
            s += 1
            p += n
    return steps


def trace_mixed(seqs: dict[str, list[int]], prompt_lens: dict[str, int], max_live: int = 4,
                portions=(13, 2, 32, 6, 3, 20), seed: int = 0) -> list[dict]:
    """Up to `max_live` requests at a time: portions of some prompts beside single decoded
    tokens of others in the same step; some requests sit a step out; a finished request is
    ended and the next one starts in the following step, on the pages it gave back."""
    import random

    rng = random.Random(seed)
    waiting = list(seqs)
    live: list[str] = []
    pos = {name: 0 for name in seqs}
    steps, s, k = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, ended = [], []
        for name in list(live):
            if len(live) > 1 and rng.random() < 0.15:
                continue  # left out of this step, goes on later
            seq, p = seqs[name], pos[name]
            if p < prompt_lens[name]:
                n = min(portions[k % len(portions)], prompt_lens[name] - p)
                k += 1
            else:
                n = 1
            entries.append(_entry(name, seq, p, n))
            pos[name] = p + n
            if pos[name] == len(seq):
                ended.append(name)
                live.remove(name)
        if not entries:
            continue
        steps.append({"step": s, "entries": entries, "end": ended})
        s += 1
    return steps


def peak_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time under `steps`, each request's count
    rounded up to a multiple of `round_to`."""
    held: dict[str, int] = {}
    peak = 0
    for rec in steps:
        for e in rec["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for name in rec["end"]:
            held.pop(name, None)
    return peak


def replay_in_process(model, steps: list[dict], num_blocks: int, block_size: int, max_requests: int = 8):
    """Drives the framework's `ModelRunner` (what bin/trace_run drives) inside this process, so that a test can
    look at the cache manager meanwhile.  Returns ({step: float32 [wanted, vocab]}, {request: set of pages it
    ever held}, the runner)."""
    from nanospec_b200.engine import ModelRunner, StepEntry

    runner = ModelRunner(model, num_blocks=num_blocks, block_size=block_size, max_requests=max_requests)
    ids: dict[str, int] = {}
    pages: dict[str, set[int]] = {}
    results = {}
    for rec in steps:
        entries = []
        for e in rec["entries"]:
            if e["id"] not in ids:
                ids[e["id"]] = len(pages)
                pages[e["id"]] = set()
                runner.begin(ids[e["id"]])
            entries.append(StepEntry(ids[e["id"]], e["tokens"], e.get("want", [])))
        out = runner.step(entries)
        if out is not None:
            results[rec["step"]] = out.float().cpu().numpy()
        for e in rec["entries"]:
            for gi in range(len(runner.manager.groups)):
                pages[e["id"]].update(p for p in runner.manager.table(gi, ids[e["id"]]) if p >= 0)
        for name in rec["end"]:
            runner.end(ids.pop(name))
        runner.manager.check()
    return results, pages, runner

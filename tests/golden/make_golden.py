"""Compares the plain implementation (tests/plain_llama.py) with the reference's own model
code, run on the CPU in float32, and records small outputs of the plain implementation.

Run once where the reference tree is present:

    python tests/golden/make_golden.py /path/to/reference

For each tiny configuration it writes a seeded random model to a temporary folder, loads it
with the reference's `load_model(folder, "cpu", float32, "sdpa")` and runs (1) one whole
prompt through `LlamaForCausalLM` over its paged cache and SDPA backend, (2) `process` and
`draw` on the last row, (3) `compute_inv_freq`.  It asserts that the plain implementation
agrees (logits within 2e-5, frequencies bit for bit, same drawn tokens) and writes
tests/golden/plain_outputs.json: per configuration the seed, the prompt, the logits of the
last position at 16 fixed vocabulary entries, the greedy tokens of 8 steps, and the largest
difference to the reference that was seen.  tests/test_plain.py checks the plain
implementation against this file, so the anchor holds where the reference is absent.
"""

from __future__ import annotations

import json
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

import plain_llama as plain  # noqa: E402
from conftest import TINY, random_ids  # noqa: E402

from nanospec_b200.weights import write_random_model  # noqa: E402


def main(reference: str) -> None:
    sys.path.insert(0, reference)
    from kv.allocator import BlockAllocator
    from kv.cache import AttnMeta, PagedKVCache
    from model.llama import compute_inv_freq
    from model.loader import load_model
    from spec.sampling import draw, process

    out = {}
    for name, spec in TINY.items():
        cfg_t = spec["config"]
        with tempfile.TemporaryDirectory() as d:
            write_random_model(d, cfg_t, seed=spec["seed"])
            ref = load_model(d, device="cpu", dtype=torch.float32, backend="sdpa")
            cfg, w = plain.read_folder(d)
        prompt = random_ids(41, cfg["vocab"], seed=100 + spec["seed"])

        # (1) whole prompt, logits at every position
        alloc = BlockAllocator(64, spec["page"])
        kv = PagedKVCache(ref.config, 64, spec["page"], "cpu", torch.float32)
        table = alloc.alloc(0, len(prompt))
        meta = AttnMeta.build([table], [len(prompt)], spec["page"], "cpu")
        ref_logits, _ = ref(torch.tensor(prompt), kv, meta)
        mine = plain.plain_forward(cfg, w, prompt)
        diff = (ref_logits - mine).abs().max().item()
        assert diff < 2e-5, (name, diff)

        # (2) frequencies
        inv_ref = compute_inv_freq(ref.config)
        inv_mine = plain.plain_inv_freq(cfg["head_dim"], cfg["theta"], cfg["scaling"])
        assert torch.equal(inv_ref, inv_mine), name

        # (3) sampling functions on the reference's last row
        z = ref_logits[-1:].clone()
        draws = []
        for temp, top_k, top_p, u in [(0.8, 0, 1.0, 0.37), (1.3, 5, 1.0, 0.81), (0.7, 0, 0.6, 0.52), (1.0, 7, 0.9, 0.05)]:
            lp_ref = process(z, torch.tensor([temp]), torch.tensor([top_k]), torch.tensor([top_p]), nucleus=True)
            tok_ref = int(draw(lp_ref, torch.zeros_like(lp_ref), torch.tensor([u]))[0])
            lp_mine = plain.plain_process(z[0], temp, top_k, top_p)
            finite = torch.isfinite(lp_ref[0])
            assert torch.equal(finite, torch.isfinite(lp_mine)), name
            assert (lp_ref[0][finite] - lp_mine[finite]).abs().max() < 1e-5
            tok_mine = plain.plain_draw(lp_mine, u)
            assert tok_ref == tok_mine, (name, tok_ref, tok_mine)
            draws.append({"temperature": temp, "top_k": top_k, "top_p": top_p, "u": u, "token": tok_mine})

        greedy, _ = plain.plain_greedy(cfg, w, prompt, 8)
        probe = list(range(0, cfg["vocab"], max(1, cfg["vocab"] // 16)))[:16]
        out[name] = {
            "seed": spec["seed"], "prompt": prompt, "probe_vocab_entries": probe,
            "last_logits_at_probe": [float(mine[-1, i]) for i in probe],
            "greedy_8": greedy, "draws": draws, "max_abs_diff_to_reference": diff,
        }
        print(f"{name}: plain vs reference max |diff| = {diff:.3g}; greedy {greedy}")
    (HERE / "plain_outputs.json").write_text(json.dumps(out, indent=1))


if __name__ == "__main__":
    # the reference's source tree: the first argument, or a folder `reference` beside this repository
    main(sys.argv[1] if len(sys.argv) > 1 else str(Path(__file__).resolve().parents[3] / "reference"))

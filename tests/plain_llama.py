"""A plain, slow implementation of the Llama 3 dense decoder: whole sequences, no cache,
float32 on the CPU, one function per part.  It shares no code with the engine (it reads the
model folder with the `safetensors` package and `json`), and every function cites the lines
of the reference it restates.  tests/golden/make_golden.py compares it once with the
reference's own model code.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


# ---------------------------------------------------------------------------------------
# configuration and weights
# ---------------------------------------------------------------------------------------
def read_folder(folder) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict with the reference's defaults applied (model/llama.py:39-78),
    and every tensor of the folder as float32 (model/loader.py:57-60)."""
    folder = Path(folder)
    raw = json.loads((folder / "config.json").read_text())
    assert raw.get("model_type") == "llama"
    rope = dict(raw.get("rope_parameters") or raw.get("rope_scaling") or {})
    theta = float(rope.pop("rope_theta", raw.get("rope_theta", 10000.0)))
    rope_type = rope.pop("rope_type", rope.pop("type", "default"))
    heads = raw["num_attention_heads"]
    cfg = {
        "vocab": raw["vocab_size"], "hidden": raw["hidden_size"], "inter": raw["intermediate_size"],
        "layers": raw["num_hidden_layers"], "heads": heads, "kv_heads": raw.get("num_key_value_heads", heads),
        "head_dim": raw.get("head_dim") or raw["hidden_size"] // heads, "eps": raw.get("rms_norm_eps", 1e-5),
        "theta": theta, "scaling": rope if rope_type == "llama3" else None,
        "tied": bool(raw.get("tie_word_embeddings", False)), "max_pos": raw["max_position_embeddings"],
    }
    weights: dict[str, torch.Tensor] = {}
    for shard in sorted(folder.glob("*.safetensors")):
        with safe_open(shard, framework="pt", device="cpu") as f:
            for name in f.keys():
                weights[name] = f.get_tensor(name).to(torch.float32)
    if "lm_head.weight" not in weights:  # model/loader.py:62-66
        assert cfg["tied"]
        weights["lm_head.weight"] = weights["model.embed_tokens.weight"]
    return cfg, weights


# ---------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------
def plain_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """model/llama.py:98-118."""
    ar = torch.arange(0, head_dim, 2, dtype=torch.int64).float()
    inv_freq = 1.0 / (theta ** (ar / head_dim))
    if scaling is None:
        return inv_freq
    factor, lo, hi = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    old = scaling["original_max_position_embeddings"]
    wavelen = 2 * math.pi / inv_freq
    out = torch.where(wavelen > old / lo, inv_freq / factor, inv_freq)
    smooth = (old / wavelen - lo) / (hi - lo)
    smoothed = (1 - smooth) * out / factor + smooth * out
    medium = ~(wavelen < old / hi) * ~(wavelen > old / lo)
    return torch.where(medium, smoothed, out)


def plain_rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """model/llama.py:92-95 (eps inside the root, plain gain)."""
    h = x.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return gain * h


def plain_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x [S, heads, d]; model/llama.py:130-136 (table), 150-158 (rotate half)."""
    freqs = torch.outer(positions.float(), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos()[:, None], emb.sin()[:, None]
    d = x.shape[-1]
    rot = torch.cat((-x[..., d // 2:], x[..., : d // 2]), dim=-1)
    return x * cos + rot * sin


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0,
                    scale: float | None = None) -> torch.Tensor:
    """q [S, nq, d], k and v [S, nkv, d], causal; query head h reads kv head h // (nq/nkv)
    (model/attention.py:22-43 with enable_gqa, scale 1/sqrt(d)).  `window` > 0 limits a
    query at position p to the keys p-window+1 .. p (no counterpart in the reference)."""
    S, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, kk) * scale
    qpos = torch.arange(S, device=q.device)[:, None]
    kpos = torch.arange(S, device=q.device)[None, :]
    mask = kpos <= qpos
    if window > 0:
        mask &= kpos > qpos - window
    scores = scores.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vv)


def plain_attention_block(x, w, prefix, cfg, positions, inv_freq, window: int = 0) -> torch.Tensor:
    """model/llama.py:173-184: projections, rope on q and k, attention, output projection."""
    S = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(S, cfg["heads"], cfg["head_dim"])
    k = (x @ w[prefix + "k_proj.weight"].T).view(S, cfg["kv_heads"], cfg["head_dim"])
    v = (x @ w[prefix + "v_proj.weight"].T).view(S, cfg["kv_heads"], cfg["head_dim"])
    q, k = plain_rope(q, positions, inv_freq), plain_rope(k, positions, inv_freq)
    o = plain_attention(q, k, v, window)
    return o.reshape(S, -1) @ w[prefix + "o_proj.weight"].T


def plain_mlp(x, w, prefix) -> torch.Tensor:
    """model/llama.py:194-195: down(silu(gate(x)) * up(x))."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return (torch.nn.functional.silu(g) * u) @ w[prefix + "down_proj.weight"].T


def plain_layer(x, w, i, cfg, positions, inv_freq) -> torch.Tensor:
    """model/llama.py:206-208."""
    p = f"model.layers.{i}."
    x = x + plain_attention_block(plain_rmsnorm(x, w[p + "input_layernorm.weight"], cfg["eps"]), w, p + "self_attn.",
                                  cfg, positions, inv_freq)
    return x + plain_mlp(plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")


def plain_forward(cfg: dict, w: dict[str, torch.Tensor], ids: list[int]) -> torch.Tensor:
    """Logits [S, vocab] at every position of one whole sequence (model/llama.py:219-232,284-286)."""
    with torch.no_grad():
        dev = w["model.embed_tokens.weight"].device  # the weights may lie on a GPU: the same arithmetic there
        t = torch.tensor(ids, dtype=torch.int64, device=dev)
        positions = torch.arange(len(ids), device=dev)
        inv_freq = plain_inv_freq(cfg["head_dim"], cfg["theta"], cfg["scaling"]).to(dev)
        x = w["model.embed_tokens.weight"][t]
        for i in range(cfg["layers"]):
            x = plain_layer(x, w, i, cfg, positions, inv_freq)
        h = plain_rmsnorm(x, w["model.norm.weight"], cfg["eps"])
        return h @ w["lm_head.weight"].T


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------
def plain_process(z: torch.Tensor, temp: float, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """One row of raw logits -> processed log-probs (spec/sampling.py:24-35)."""
    z = z / (temp if temp > 0 else 1.0)
    if top_k > 0 or top_p < 1.0:
        srt, idx = z.sort(-1, descending=True)
        p = srt.softmax(-1)
        keep = (p.cumsum(-1) - p) <= top_p
        if top_k > 0:
            keep &= torch.arange(z.shape[-1]) < top_k
        z = torch.full_like(z, float("-inf")).scatter_(-1, idx, srt.masked_fill(~keep, float("-inf")))
    return z.log_softmax(-1)


def plain_draw(lp: torch.Tensor, u: float) -> int:
    """Inverse-CDF draw in vocabulary order (spec/sampling.py:38-42 with q = 0)."""
    cdf = lp.exp().cumsum(-1)
    t = torch.searchsorted(cdf, torch.tensor([u * cdf[-1].item()]), right=True)
    return int(min(int(t), lp.shape[-1] - 1))


def plain_greedy(cfg, w, prompt: list[int], n_new: int) -> tuple[list[int], list[torch.Tensor]]:
    """Greedy continuation by re-running the whole sequence for every token
    (argmax of raw logits, engine/engine.py:385,399).  Returns tokens and each step's logits."""
    ids, out, rows = list(prompt), [], []
    for _ in range(n_new):
        z = plain_forward(cfg, w, ids)[-1]
        tok = int(z.argmax())
        out.append(tok)
        rows.append(z)
        ids.append(tok)
    return out, rows

"""Random-weights mode: writes a model folder (config.json + model.safetensors) from a
configuration and a seed, or fills a model in place on its device.

Matrices and embeddings are N(0, 0.02) and norm gains 1 + N(0, 0.1), drawn on the CPU from
one `torch.Generator` seeded with `seed`, tensor by tensor in name order, so a folder is
reproducible.  Values are rounded to bfloat16 before they are stored: the float32 path and the
bfloat16 path then read the very same numbers, and a difference between them is never a
difference of weights.  The reference has no such mode (its tests download a checkpoint,
tests/conftest.py:16).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..parts.base import WeightSpec
from .loader import build_model
from .safetensors_io import write_safetensors


def _draw(spec: WeightSpec, gen: torch.Generator, device="cpu") -> torch.Tensor:
    if spec.rule == "int32":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    t = torch.empty(spec.shape, dtype=torch.float32, device=device).normal_(0.0, 1.0, generator=gen)
    if spec.init == "gain":
        t = 1.0 + 0.1 * t
    else:
        t = spec.std * t
    return t.to(torch.bfloat16)


def write_random_model(folder: str | Path, config, seed: int = 0, generation_config: dict | None = None) -> Path:
    """`config`: a typed configuration with `to_hf()` (e.g. LlamaConfig) or a config.json dict."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg_json = config if isinstance(config, dict) else config.to_hf()
    model, _ = build_model(cfg_json, generation_config, torch.float32, "cpu")
    gen = torch.Generator().manual_seed(int(seed))
    tensors = {}
    for name, spec in sorted(model.weight_specs().items()):
        if spec.alias is not None:
            continue  # a tied head is stored once, under the embedding's name
        tensors[name] = _draw(spec, gen)
    (folder / "config.json").write_text(json.dumps(cfg_json, indent=2))
    if generation_config:
        (folder / "generation_config.json").write_text(json.dumps(generation_config, indent=2))
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": str(seed)})
    return folder


def random_model(config, seed: int = 0, device="cuda", dtype: torch.dtype = torch.bfloat16, return_tensors: bool = False):
    """A model with random weights drawn directly on `device` (no files): for benchmarks at
    sizes where writing the folder first would only cost time.  Same distributions as
    `write_random_model`, but the device's generator, so not the same numbers.  With
    `return_tensors` the checkpoint-named tensors are returned beside the model, so that an
    oracle can compute with the very weights the engine holds."""
    cfg_json = config if isinstance(config, dict) else config.to_hf()
    model, _ = build_model(cfg_json, None, dtype, device)
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(int(seed))
    tensors: dict[str, torch.Tensor] = {}
    specs = model.weight_specs()
    for name, spec in sorted(specs.items()):
        if spec.alias is not None:
            continue
        t = _draw(spec, gen, device=dev)
        tensors[name] = t.to(torch.int32 if spec.rule == "int32" else torch.float32 if spec.rule == "float32" else dtype)
    for name, spec in specs.items():
        if spec.alias is not None:
            tensors[name] = tensors[spec.alias]
    model.bind(tensors)
    return (model, tensors) if return_tensors else model

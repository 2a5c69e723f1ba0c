"""From a model folder (config.json + *.safetensors) to a `DecoderModel` with its weights.

Tensors are bound by name.  The reference loads with `strict=True` (model/loader.py:57-70):
a missing or unexpected tensor, or a wrong shape, is an error; a checkpoint without a head
is accepted only when the configuration ties the head to the embedding.  Here all such
faults of a folder are collected and raised as one `WeightError`.

Precision: matrices are held in the run's dtype (bfloat16 for serving, float32 for the exact
path), small float tensors that the kernels read as float32 (norm gains) stay float32, and
integer tables are int32.
"""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.files import read_config_files
from ..config.registry import resolve_architecture
from ..parts.base import WeightSpec
from ..parts.model import DecoderModel
from .safetensors_io import SafetensorsFile, iter_model_files


class WeightError(ValueError):
    """The tensors of a model folder do not fit the model: lists missing and unexpected
    names and wrong shapes."""

    def __init__(self, folder, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected, self.wrong_shape, self.other = list(missing), list(unexpected), list(wrong_shape), list(other)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        lines.extend(f"  {o}" for o in self.other)
        super().__init__("\n".join(lines))


def _cast(t: torch.Tensor, spec: WeightSpec, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    if spec.rule == "int32":
        return t.to(device=device, dtype=torch.int32)
    if spec.rule == "float32":
        return t.to(device=device, dtype=torch.float32)
    return t.to(device=device, dtype=dtype)


def build_model(cfg_json: dict, generation_json: dict | None, dtype: torch.dtype, device) -> tuple[DecoderModel, object]:
    """The (unbound) model that a config.json asks for, and its typed configuration."""
    from .. import architectures  # noqa: F401  (registers the built-in architectures)

    arch = resolve_architecture(cfg_json)
    config = arch.config_from_hf(cfg_json, generation_json)
    model = DecoderModel(arch.recipe(config), dtype, torch.device(device))
    model.config = config
    return model, config


def load_model(folder: str | Path, device: str | torch.device = "cuda", dtype: torch.dtype = torch.bfloat16,
               backend: str = "auto") -> DecoderModel:
    """Counterpart of the reference's `load_model(model, device, dtype, backend)` (model/loader.py:41-83)
    for a local folder.  `backend` is taken so that a call written for the reference still reads; there
    is one execution path here (this package's CUDA kernels), so anything but "auto" is refused."""
    if backend != "auto":
        raise ValueError(f"backend={backend!r}: this engine has one execution path, its own CUDA kernels; pass \"auto\"")
    folder = Path(folder)
    cfg_json, gen_json = read_config_files(folder)
    model, _ = build_model(cfg_json, gen_json, dtype, device)
    specs = model.weight_specs()

    files = [SafetensorsFile(p) for p in iter_model_files(folder)]
    if not files:
        raise WeightError(folder, sorted(specs), [], [], other=["no *.safetensors file in the folder"])
    where: dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.keys():
            where[name] = f

    missing, wrong = [], []
    source: dict[str, str] = {}
    for name, spec in specs.items():
        src = name if name in where else (spec.alias if spec.alias in where else None)
        if src is None:
            missing.append(name if not spec.alias else f"{name} (nor its tied source {spec.alias})")
            continue
        source[name] = src
        got = where[src].shape(src)
        if tuple(got) != tuple(spec.shape):
            wrong.append((src, got, spec.shape))
    unexpected = sorted(set(where) - set(source.values()) - set(specs))
    if missing or unexpected or wrong:
        raise WeightError(folder, sorted(missing), unexpected, wrong)

    dev = torch.device(device)
    tensors: dict[str, torch.Tensor] = {}
    by_source: dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        src = source[name]
        if src not in by_source:  # a tied head shares the embedding's tensor
            by_source[src] = _cast(where[src].tensor(src), specs.get(src, spec), dtype, dev)
        tensors[name] = by_source[src]
    model.bind(tensors)
    for f in files:
        f.close()
    return model

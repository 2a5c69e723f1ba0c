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


def update_weights(model: DecoderModel, state: dict[str, torch.Tensor]) -> None:
    """Replaces weights of a bound model in place (captured CUDA graphs and tensor maps keep pointing at the same
    memory), the reference's `Engine.update_weights` (engine/engine.py:167-176 there) for this engine's packed
    tensors.  `state`: checkpoint name -> tensor, any device and floating type.  A part that packs several
    checkpoint tensors into one (q/k/v; gate/up) takes all of its tensors or none; names the model does not have and
    wrong shapes are refused before anything is written."""
    if not model.bound:
        raise RuntimeError("the model has no weights bound")
    specs = model.weight_specs()
    unknown = sorted(set(state) - set(specs))
    wrong = [(n, tuple(t.shape), specs[n].shape) for n, t in state.items() if n in specs and tuple(t.shape) != tuple(specs[n].shape)]
    if unknown or wrong:
        raise WeightError("update_weights", [], unknown, wrong)
    for name, spec in specs.items():  # a head that shares the embedding's tensor is replaced through the embedding
        if name in state and spec.alias is not None and spec.alias not in state:
            head, table = getattr(model.head, "weight", None), getattr(model.embedding, "table", None)
            if head is not None and table is not None and head.data_ptr() == table.data_ptr():
                raise WeightError("update_weights", [], [], [], other=[f"{name} is tied to {spec.alias}: replace that tensor"])
    jobs = []
    for prefix, part in model._named_parts():
        names = list(part.weight_specs())
        given = [n for n in names if prefix + n in state]
        if not given:
            continue
        if len(given) != len(names):
            lacking = [prefix + n for n in names if n not in given]
            raise WeightError("update_weights", lacking, [], [], other=[f"the tensors under {prefix} are packed together and are replaced together"])
        jobs.append((prefix, part, names))
    for prefix, part, names in jobs:
        shadow = type(part)(part.spec, model.dtype, model.device)
        shadow.bind({n: _cast(state[prefix + n], part.weight_specs()[n], model.dtype, model.device) for n in names})
        _copy_tensors(part, shadow, prefix)


def _copy_tensors(live, shadow, where: str) -> None:
    """Every tensor that binding gave the shadow goes into the live part's tensor of the same name."""
    from ..parts.base import Part

    for attr, val in vars(shadow).items():
        if isinstance(val, torch.Tensor):
            target = getattr(live, attr, None)
            if not isinstance(target, torch.Tensor) or target.shape != val.shape or target.dtype != val.dtype:
                raise RuntimeError(f"{where}: the bound tensor {attr!r} cannot be replaced in place")
            target.copy_(val)
        elif isinstance(val, Part) and isinstance(getattr(live, attr, None), Part):
            _copy_tensors(getattr(live, attr), val, where)


"""Weights: the safetensors reader and writer, binding by name, the one error that lists
everything wrong with a folder, and the random-weights mode (no GPU)."""

from __future__ import annotations

import json
import shutil

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from nanospec_b200.weights import SafetensorsError, SafetensorsFile, WeightError, load_model, write_random_model, write_safetensors
from conftest import TINY


def test_writer_is_read_by_the_safetensors_package_and_back(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {"a.weight": torch.randn(3, 5, generator=g).to(torch.bfloat16), "b": torch.randn(7, generator=g),
               "ids": torch.arange(6, dtype=torch.int32).view(2, 3), "empty": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", tensors, {"note": "t"})
    with safe_open(tmp_path / "x.safetensors", framework="pt") as f:
        assert sorted(f.keys()) == sorted(tensors)
        for k in tensors:
            assert torch.equal(f.get_tensor(k), tensors[k])
    save_file(tensors, str(tmp_path / "y.safetensors"))
    mine = SafetensorsFile(tmp_path / "y.safetensors")
    for k, t in tensors.items():
        assert mine.shape(k) == tuple(t.shape) and mine.dtype(k) == t.dtype and torch.equal(mine.tensor(k), t)


def test_truncated_and_broken_files_are_refused(tmp_path):
    write_safetensors(tmp_path / "x.safetensors", {"a": torch.ones(4, 4)})
    raw = (tmp_path / "x.safetensors").read_bytes()
    (tmp_path / "cut.safetensors").write_bytes(raw[:-8])
    with pytest.raises(SafetensorsError, match="does not match its byte range"):
        SafetensorsFile(tmp_path / "cut.safetensors")
    (tmp_path / "short.safetensors").write_bytes(raw[:4])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(tmp_path / "short.safetensors")


def test_random_folder_is_reproducible_and_loads(tiny_folders, tmp_path):
    a2 = write_random_model(tmp_path / "again", TINY["A"]["config"], seed=TINY["A"]["seed"])
    assert (a2 / "model.safetensors").read_bytes() == (tiny_folders["A"] / "model.safetensors").read_bytes()
    other = write_random_model(tmp_path / "other", TINY["A"]["config"], seed=5)
    assert (other / "model.safetensors").read_bytes() != (a2 / "model.safetensors").read_bytes()
    m = load_model(tiny_folders["A"], device="cpu", dtype=torch.bfloat16)
    assert m.blocks[0].mixer.w_qkv.dtype == torch.bfloat16 and m.blocks[0].mixer.w_qkv.shape == (64 + 2 * 16, 64)
    assert m.blocks[0].norm_mixer.gain.dtype == torch.float32  # small float tensors are held in 32-bit
    assert m.head.weight is m.embedding.table  # tied: one tensor
    with SafetensorsFile(tiny_folders["A"] / "model.safetensors") as f:
        assert "lm_head.weight" not in f.keys()
        gains = f.tensor("model.norm.weight").float()
        assert abs(float(gains.mean()) - 1.0) < 0.1 and 0.03 < float(gains.std()) < 0.2
        w = f.tensor("model.layers.0.mlp.up_proj.weight").float()
        assert abs(float(w.std()) - 0.02) < 0.004
    b = load_model(tiny_folders["B"], device="cpu", dtype=torch.float32, backend="auto")  # the reference's fourth argument
    assert b.head.weight is not b.embedding.table and b.head.weight.dtype == torch.float32
    with pytest.raises(ValueError, match="one execution path"):
        load_model(tiny_folders["B"], device="cpu", backend="sdpa")


def _resave(folder, out, change):
    out.mkdir()
    shutil.copy(folder / "config.json", out / "config.json")
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {k: f.tensor(k).clone() for k in f.keys()}
    change(tensors)
    write_safetensors(out / "model.safetensors", tensors)
    return out


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tiny_folders, tmp_path):
    def change(t):
        del t["model.layers.1.mlp.down_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.7.extra.weight"] = torch.zeros(2)
        t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(3, 128, dtype=torch.bfloat16)

    bad = _resave(tiny_folders["B"], tmp_path / "bad", change)
    with pytest.raises(WeightError) as e:
        load_model(bad, device="cpu", dtype=torch.float32)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (3, 128), (32, 128))]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "[3, 128]", "[32, 128]"):
        assert word in text


def test_untied_model_without_head_is_an_error_and_tied_one_may_carry_a_head(tiny_folders, tmp_path):
    no_head = _resave(tiny_folders["B"], tmp_path / "nohead", lambda t: t.pop("lm_head.weight"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_model(no_head, device="cpu", dtype=torch.float32)

    def add_head(t):
        t["lm_head.weight"] = t["model.embed_tokens.weight"].clone() * 2

    with_head = _resave(tiny_folders["A"], tmp_path / "withhead", add_head)
    m = load_model(with_head, device="cpu", dtype=torch.float32)
    assert torch.equal(m.head.weight, m.embedding.table * 2)


def test_empty_folder_and_unknown_architecture(tmp_path, tiny_folders):
    (tmp_path / "e").mkdir()
    shutil.copy(tiny_folders["A"] / "config.json", tmp_path / "e" / "config.json")
    with pytest.raises(WeightError, match="no \\*.safetensors"):
        load_model(tmp_path / "e", device="cpu", dtype=torch.float32)
    cfg = json.loads((tiny_folders["A"] / "config.json").read_text())
    cfg["architectures"] = ["NopeForCausalLM"]
    (tmp_path / "e" / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(ValueError, match="unknown architecture"):
        load_model(tmp_path / "e", device="cpu", dtype=torch.float32)


def test_sharded_folder(tiny_folders, tmp_path):
    out = tmp_path / "sharded"
    out.mkdir()
    shutil.copy(tiny_folders["C"] / "config.json", out / "config.json")
    with SafetensorsFile(tiny_folders["C"] / "model.safetensors") as f:
        names = sorted(f.keys())
        half = len(names) // 2
        write_safetensors(out / "model-00001-of-00002.safetensors", {k: f.tensor(k).clone() for k in names[:half]})
        write_safetensors(out / "model-00002-of-00002.safetensors", {k: f.tensor(k).clone() for k in names[half:]})
    a = load_model(out, device="cpu", dtype=torch.float32)
    b = load_model(tiny_folders["C"], device="cpu", dtype=torch.float32)
    assert torch.equal(a.blocks[0].feed_forward.w_gate_up, b.blocks[0].feed_forward.w_gate_up)

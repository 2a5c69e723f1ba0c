"""Shared test set-up: the `gpu` marker, three tiny Llama configurations that differ in
every size and option, and model folders with seeded random weights written to a temporary
folder (never committed)."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from nanospec_b200.config import Llama3RopeScaling, LlamaConfig  # noqa: E402
from nanospec_b200.weights import write_random_model  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny A and B are the two tiny configurations of the benchmark description; C adds sizes
# that are no power of two anywhere (width, heads, vocabulary) and a page of 4.
TINY = {
    "A": dict(
        config=LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                           num_attention_heads=8, num_key_value_heads=2, head_dim=8, rms_norm_eps=1e-5,
                           rope_theta=10000.0, max_position_embeddings=256, rope_scaling=None,
                           tie_word_embeddings=True, eos_token_ids=()),
        page=16, seed=11),
    "B": dict(
        config=LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=352, num_hidden_layers=3,
                           num_attention_heads=4, num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-6,
                           rope_theta=500000.0, max_position_embeddings=512,
                           rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 64), tie_word_embeddings=False,
                           eos_token_ids=()),
        page=8, seed=22),
    "C": dict(
        config=LlamaConfig(vocab_size=331, hidden_size=96, intermediate_size=200, num_hidden_layers=1,
                           num_attention_heads=6, num_key_value_heads=3, head_dim=16, rms_norm_eps=1e-4,
                           rope_theta=1000000.0, max_position_embeddings=384,
                           rope_scaling=Llama3RopeScaling(4.0, 1.0, 2.0, 32), tie_word_embeddings=False,
                           eos_token_ids=()),
        page=4, seed=33),
}


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory) -> dict[str, Path]:
    out = {}
    for name, spec in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(d, spec["config"], seed=spec["seed"])
        out[name] = d
    return out


# Two-layer models at real layer widths, which select the kernels that the tiny ones never reach (TMA decode
# attention in a cluster, tcgen05 prefill attention, the products' gated, norm and rotation epilogues):
# "wide128" has the benchmark configuration's widths, "wide64" those of its smallest sibling with heads of 64 and
# a tied head.  Vocabularies are no power of two.
WIDE = {
    "wide128": LlamaConfig(vocab_size=20011, hidden_size=4096, intermediate_size=14336, num_hidden_layers=2,
                           num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                           max_position_embeddings=1024, rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 256),
                           tie_word_embeddings=True),
    "wide64": LlamaConfig(vocab_size=10007, hidden_size=2048, intermediate_size=8192, num_hidden_layers=2,
                          num_attention_heads=32, num_key_value_heads=8, head_dim=64, rms_norm_eps=1e-5, rope_theta=500000.0,
                          max_position_embeddings=1024, rope_scaling=Llama3RopeScaling(32.0, 1.0, 4.0, 256),
                          tie_word_embeddings=True),
}


@pytest.fixture(scope="session")
def wide_folders(tmp_path_factory) -> dict[str, Path]:
    out = {}
    for i, (name, cfg) in enumerate(WIDE.items()):
        d = tmp_path_factory.mktemp(name)
        write_random_model(d, cfg, seed=21 + i)
        out[name] = d
    return out


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

"""Configuration and registry (no GPU)."""

from __future__ import annotations

import json

import pytest

from nanospec_b200 import architectures  # noqa: F401
from nanospec_b200.config import (ConfigError, EngineConfig, Llama3RopeScaling, LlamaConfig, ModelRecipe, PartSpec, Run,
                                  registered_architectures, resolve_architecture)
from nanospec_b200.architectures.llama import llama_recipe
from conftest import TINY

BASE = {"model_type": "llama", "vocab_size": 100, "hidden_size": 48, "intermediate_size": 96, "num_hidden_layers": 2,
        "num_attention_heads": 6, "max_position_embeddings": 128}


def test_defaults_follow_the_reference():
    c = LlamaConfig.from_hf(BASE)
    assert (c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.rope_theta) == (6, 8, 1e-5, 10000.0)
    assert c.rope_scaling is None and not c.tie_word_embeddings and c.eos_token_ids == ()
    assert (c.q_size, c.kv_size, c.group_size) == (48, 48, 1)


def test_rope_blocks_old_and_new_spelling():
    block = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
             "original_max_position_embeddings": 64}
    old = LlamaConfig.from_hf({**BASE, "rope_theta": 500000.0, "rope_scaling": block})
    new = LlamaConfig.from_hf({**BASE, "rope_parameters": {**block, "rope_theta": 500000.0}})
    legacy = LlamaConfig.from_hf({**BASE, "rope_theta": 500000.0, "rope_scaling": {**{k: v for k, v in block.items() if k != "rope_type"}, "type": "llama3"}})
    assert old == new == legacy
    assert old.rope_scaling == Llama3RopeScaling(8.0, 1.0, 4.0, 64) and old.rope_theta == 500000.0


def test_eos_from_generation_config_wins():
    assert LlamaConfig.from_hf({**BASE, "eos_token_id": 7}).eos_token_ids == (7,)
    assert LlamaConfig.from_hf({**BASE, "eos_token_id": 7}, {"eos_token_id": [8, 9]}).eos_token_ids == (8, 9)


@pytest.mark.parametrize("change,word", [
    ({"model_type": "mistral"}, "not a llama config"),
    ({"attention_bias": True}, "biased"),
    ({"mlp_bias": True}, "biased"),
    ({"hidden_act": "gelu"}, "silu"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "unsupported rope_type"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "lacks"),
    ({"num_key_value_heads": 4}, "not a multiple"),
    ({"head_dim": 7}, "even"),
    ({"num_hidden_layers": 0}, "positive"),
])
def test_refusals(change, word):
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_hf({**BASE, **change})


def test_missing_keys_are_listed():
    cfg = {k: v for k, v in BASE.items() if k not in ("vocab_size", "intermediate_size")}
    with pytest.raises(ConfigError, match="vocab_size, intermediate_size"):
        LlamaConfig.from_hf(cfg)


@pytest.mark.parametrize("name", list(TINY))
def test_round_trip_through_config_json(name):
    c = TINY[name]["config"]
    assert LlamaConfig.from_hf(json.loads(json.dumps(c.to_hf()))) == c


def test_registry_picks_by_architecture_name_then_model_type():
    assert "LlamaForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"}).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError, match="unknown architecture 'FooForCausalLM'.*LlamaForCausalLM"):
        resolve_architecture({"architectures": ["FooForCausalLM"], "model_type": "llama"})


def test_recipe_carries_every_size_as_a_parameter():
    c = TINY["B"]["config"]
    r = llama_recipe(c)
    assert len(r.layers) == 3 and [run.layer for run in r.order] == [0, 1, 2] and r.num_lanes == 3
    m = r.layers[1].mixer
    assert (m.kind, m["heads"], m["kv_heads"], m["head_dim"], m["hidden"]) == ("gqa_attention", 4, 1, 32, 128)
    assert m["position"].kind == "rope" and m["position"]["theta"] == 500000.0 and m["position"]["scaling"]["factor"] == 8.0
    assert r.layers[0].feed_forward["intermediate"] == 352 and r.layers[0].norm["eps"] == 1e-6
    assert r.head["tied_to"] is None and llama_recipe(TINY["A"]["config"]).head["tied_to"] == "model.embed_tokens.weight"


def test_order_is_data_and_is_checked():
    c = TINY["A"]["config"]
    r = llama_recipe(c)
    kw = dict(architecture="x", embedding=r.embedding, layers=r.layers, final_norm=r.final_norm,
              final_norm_prefix=r.final_norm_prefix, head=r.head, vocab_size=256, hidden_size=64, max_positions=256)
    # a layer named twice, and a run that reads another run's lane
    ok = ModelRecipe(order=(Run(0, 0), Run(1, 1), Run(0, 2), Run(1, 1, writes=False)), **kw)
    assert ok.num_lanes == 3
    with pytest.raises(ValueError, match="names layer 5"):
        ModelRecipe(order=(Run(5, 0),), **kw)
    with pytest.raises(ValueError, match="already writes"):
        ModelRecipe(order=(Run(0, 0), Run(1, 0)), **kw)
    with pytest.raises(ValueError, match="before any run has written"):
        ModelRecipe(order=(Run(0, 1, writes=False),), **kw)
    with pytest.raises(ValueError, match="numbered 0..n-1"):
        ModelRecipe(order=(Run(0, 0), Run(1, 2)), **kw)


def test_engine_config_names_and_checks():
    e = EngineConfig(num_blocks=8)
    assert (e.block_size, e.max_admit, e.max_running, e.cuda_graphs, e.record_logits, e.profile, e.head_chunk) == \
        (16, 32, None, True, False, False, 256)
    with pytest.raises(ValueError):
        EngineConfig(num_blocks=0)
    with pytest.raises(ValueError):
        EngineConfig(num_blocks=4, admission="greedy")


def test_part_spec_is_read_only():
    p = PartSpec("rmsnorm", {"hidden": 4, "eps": 1e-5})
    with pytest.raises(TypeError):
        p.params["hidden"] = 5

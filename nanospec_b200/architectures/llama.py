"""The Llama 3 dense decoder as a recipe: every layer is a pre-norm block of grouped-query
attention with rotary positions and a SwiGLU feed-forward (model/llama.py:161-254), tensor
names in the Hugging Face layout (model/llama.py:168-171,190-192,201-204,214-216,261-262)."""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.recipe import LayerSpec, ModelRecipe, PartSpec, Run
from ..config.registry import Architecture, register_architecture


def llama_recipe(cfg: LlamaConfig) -> ModelRecipe:
    scaling = None
    if cfg.rope_scaling is not None:
        s = cfg.rope_scaling
        scaling = {"factor": s.factor, "low_freq_factor": s.low_freq_factor, "high_freq_factor": s.high_freq_factor,
                   "original_max_position_embeddings": s.original_max_position_embeddings}
    position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling})
    mixer = PartSpec("gqa_attention", {
        "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim, "window": 0, "position": position,
    })
    feed_forward = PartSpec("swiglu", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size})
    norm = PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    names = {"mixer": "self_attn.", "feed_forward": "mlp.", "norm_mixer": "input_layernorm.",
             "norm_feed_forward": "post_attention_layernorm."}
    layers = tuple(
        LayerSpec(block="prenorm", prefix=f"model.layers.{i}.", mixer=mixer, feed_forward=feed_forward, norm=norm,
                  names=names)
        for i in range(cfg.num_hidden_layers))
    return ModelRecipe(
        architecture=cfg.architecture,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "name": "model.embed_tokens"}),
        layers=layers,
        order=tuple(Run(layer=i, lane=i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm,
        final_norm_prefix="model.norm.",
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "name": "lm_head",
                                 "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None}),
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        eos_token_ids=cfg.eos_token_ids,
    )


LLAMA = register_architecture(Architecture(
    name="LlamaForCausalLM", model_type="llama", config_from_hf=LlamaConfig.from_hf, recipe=llama_recipe))

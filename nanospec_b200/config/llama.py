"""Typed configuration of the Llama 3 dense decoder, read from its own config.json keys.

Keys, defaults and refusals follow the reference's `LlamaConfig.from_hf`
(model/llama.py:22-78): `model_type` must be "llama", biased projections are refused (here also
an activation other than silu, which the reference would run as silu without a word),
`rope_parameters` (newer writers) or `rope_theta` + `rope_scaling` (older writers) give
the rotary constants, only the rope types "default" and "llama3" are known, `head_dim`
defaults to hidden_size // num_attention_heads, `num_key_value_heads` to the head count,
`rms_norm_eps` to 1e-5, and `eos_token_id` of generation_config.json wins over config.json.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .files import ConfigError


@dataclass(frozen=True)
class Llama3RopeScaling:
    """The `rope_type == "llama3"` block: wavelength-banded rescale of the frequencies."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_hf(self) -> dict[str, Any]:
        return {
            "rope_type": "llama3",
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "max_position_embeddings",
)


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    rope_scaling: Llama3RopeScaling | None = None
    tie_word_embeddings: bool = False
    bos_token_id: int | None = None
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    architecture = "LlamaForCausalLM"
    model_type = "llama"

    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotate-half RoPE")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")

    # sizes that follow from the keys
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_hf(cls, cfg: dict[str, Any], generation_cfg: dict[str, Any] | None = None) -> "LlamaConfig":
        if cfg.get("model_type") != "llama":
            raise ConfigError(f"not a llama config: model_type={cfg.get('model_type')!r}")
        if cfg.get("attention_bias") or cfg.get("mlp_bias"):
            raise ConfigError("biased projections are not supported")
        if cfg.get("hidden_act", "silu") != "silu":  # the reference applies silu whatever the key says (model/llama.py:195)
            raise ConfigError(f"the gated feed-forward applies silu; hidden_act={cfg['hidden_act']!r} is not supported")
        missing = [k for k in _REQUIRED if k not in cfg]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {', '.join(missing)}")

        rope = dict(cfg.get("rope_parameters") or cfg.get("rope_scaling") or {})
        rope_theta = float(rope.pop("rope_theta", cfg.get("rope_theta", 10000.0)))
        rope_type = rope.pop("rope_type", rope.pop("type", "default"))
        if rope_type == "default":
            scaling = None
        elif rope_type == "llama3":
            try:
                scaling = Llama3RopeScaling(
                    factor=float(rope["factor"]),
                    low_freq_factor=float(rope["low_freq_factor"]),
                    high_freq_factor=float(rope["high_freq_factor"]),
                    original_max_position_embeddings=int(rope["original_max_position_embeddings"]),
                )
            except KeyError as e:
                raise ConfigError(f"llama3 rope block lacks {e.args[0]!r}") from None
        else:
            raise ConfigError(f"unsupported rope_type {rope_type!r}")

        heads = cfg["num_attention_heads"]
        eos = cfg.get("eos_token_id")
        if generation_cfg and generation_cfg.get("eos_token_id") is not None:
            eos = generation_cfg["eos_token_id"]
        if isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),) if eos is not None else ()

        return cls(
            vocab_size=cfg["vocab_size"],
            hidden_size=cfg["hidden_size"],
            intermediate_size=cfg["intermediate_size"],
            num_hidden_layers=cfg["num_hidden_layers"],
            num_attention_heads=heads,
            num_key_value_heads=cfg.get("num_key_value_heads") or heads,
            head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
            rope_theta=rope_theta,
            max_position_embeddings=cfg["max_position_embeddings"],
            rope_scaling=scaling,
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            bos_token_id=cfg.get("bos_token_id"),
            eos_token_ids=eos_ids,
        )

    def to_hf(self) -> dict[str, Any]:
        """The config.json that `from_hf` reads back to an equal configuration."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
            "hidden_act": "silu",
        }
        if self.rope_scaling is not None:
            out["rope_scaling"] = self.rope_scaling.to_hf()
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out

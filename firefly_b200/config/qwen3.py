"""Typed configuration of Qwen3 dense (``Qwen3ForCausalLM``).

Keys, meanings and defaults are those the reference reads from ``config.json``
(src/server.cu:45-63): the ten sizes and constants below, with
``num_key_value_heads`` defaulting to ``num_attention_heads`` and ``head_dim`` to
``hidden_size / num_attention_heads``.  The reference never reads
``tie_word_embeddings`` and fails on checkpoints without ``lm_head.weight``
(src/model/qwen_model.cu:92); here the key is honoured.  Keys that would change
the arithmetic and that the reference's model does not implement are refused by
name instead of being ignored.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Mapping

from .base import ConfigError, ModelConfig


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    architecture: ClassVar[str] = "Qwen3ForCausalLM"

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        g = cls._get
        hidden = g(raw, "hidden_size", int)
        n_heads = g(raw, "num_attention_heads", int)
        if n_heads <= 0:
            raise ConfigError("config.json: 'num_attention_heads' must be positive")
        if "head_dim" not in raw or raw["head_dim"] is None:
            if hidden % n_heads:
                raise ConfigError(
                    f"config.json: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {n_heads}")
        cfg = cls(
            hidden_size=hidden,
            intermediate_size=g(raw, "intermediate_size", int),
            num_hidden_layers=g(raw, "num_hidden_layers", int),
            num_attention_heads=n_heads,
            num_key_value_heads=g(raw, "num_key_value_heads", int, n_heads),
            head_dim=g(raw, "head_dim", int, hidden // n_heads),
            vocab_size=g(raw, "vocab_size", int),
            max_position_embeddings=g(raw, "max_position_embeddings", int, 32768),
            rms_norm_eps=g(raw, "rms_norm_eps", float, 1e-6),
            rope_theta=g(raw, "rope_theta", float, 10000.0),
            tie_word_embeddings=g(raw, "tie_word_embeddings", bool, False),
        )
        # what would change the arithmetic and is not part of this architecture's model
        if g(raw, "attention_bias", bool, False):
            raise ConfigError("config.json: attention_bias=true is not supported "
                              "(Qwen3 dense binds no bias tensors)")
        if g(raw, "use_sliding_window", bool, False):
            raise ConfigError("config.json: use_sliding_window=true is not supported by "
                              "Qwen3ForCausalLM in this engine")
        lt = raw.get("layer_types")
        if lt is not None and any(t != "full_attention" for t in lt):
            raise ConfigError("config.json: layer_types other than 'full_attention' are not supported "
                              "(every Qwen3 dense layer attends to all earlier tokens)")
        if raw.get("rope_scaling") is not None:
            raise ConfigError("config.json: rope_scaling is not supported "
                              "(plain rotary position encoding only)")
        act = g(raw, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (silu only)")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            v = getattr(self, key)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"config.json: '{key}' must be a positive integer, got {v!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary encoding")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"config.json: rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"config.json: rope_theta must be > 0, got {self.rope_theta}")

"""Typed configuration of dense Qwen3, read from its own config.json keys.

The keys are those of the fixture in crates/models/src/qwen3.rs:136-156; the dispatch
guard (`Qwen3ForCausalLM` / `qwen3`, anything else rejected with both names in the
message) follows qwen3.rs:31-36.  Validation of head counts follows
crates/models/src/components/gated_attention.rs:36-62 and of the rotary width
crates/models/src/components/rope.rs:22-46.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

from .errors import InvalidConfig
from .metadata import ModelMetadata, metadata_from_json

ARCHITECTURE = "Qwen3ForCausalLM"
MODEL_TYPE = "qwen3"


def _integer(raw: dict, key: str, default=None) -> int:
    value = raw.get(key, default)
    if value is None:
        raise InvalidConfig(f"config.json must include {key!r}")
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise InvalidConfig(f"config.json: {key!r} must be a positive integer, found {value!r}")
    return value


def _number(raw: dict, key: str) -> float:
    value = raw.get(key)
    if value is None:
        raise InvalidConfig(f"config.json must include {key!r}")
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or value <= 0:
        raise InvalidConfig(f"config.json: {key!r} must be a finite positive number, found {value!r}")
    return float(value)


def _flag(raw: dict, key: str, default: bool) -> bool:
    value = raw.get(key, default)
    if value is None:
        return default
    if not isinstance(value, bool):
        raise InvalidConfig(f"config.json: {key!r} must be true or false, found {value!r}")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    attention_bias: bool
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    declared_dtype: Optional[str] = None

    architecture = ARCHITECTURE
    model_type = MODEL_TYPE

    def __post_init__(self):
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise InvalidConfig(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2 != 0:
            raise InvalidConfig(f"head_dim ({self.head_dim}) must be even for rotary pairs")

    @classmethod
    def from_json(cls, raw: dict) -> "Qwen3Config":
        metadata: ModelMetadata = metadata_from_json(raw)
        if (metadata.architecture, metadata.model_type) != (ARCHITECTURE, MODEL_TYPE):
            raise InvalidConfig(
                f"expected dense {ARCHITECTURE}/{MODEL_TYPE}, found {metadata.architecture}/{metadata.model_type}"
            )
        heads = _integer(raw, "num_attention_heads")
        hidden = _integer(raw, "hidden_size")
        if raw.get("head_dim") is None and hidden % heads != 0:
            raise InvalidConfig("config.json has no head_dim and hidden_size is not a multiple of num_attention_heads")
        activation = raw.get("hidden_act", "silu")
        if activation != "silu":
            raise InvalidConfig(f"hidden_act {activation!r} is not supported; dense Qwen3 uses 'silu'")
        if raw.get("rope_scaling") is not None:
            raise InvalidConfig("rope_scaling is not supported")
        if _flag(raw, "use_sliding_window", False):
            raise InvalidConfig("use_sliding_window=true is not supported: dense Qwen3 runs full causal attention")
        return cls(
            vocab_size=_integer(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_integer(raw, "intermediate_size"),
            num_hidden_layers=_integer(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=_integer(raw, "num_key_value_heads", heads),
            head_dim=_integer(raw, "head_dim", hidden // heads),
            attention_bias=_flag(raw, "attention_bias", False),
            rms_norm_eps=_number(raw, "rms_norm_eps"),
            rope_theta=_number(raw, "rope_theta"),
            max_position_embeddings=_integer(raw, "max_position_embeddings"),
            tie_word_embeddings=_flag(raw, "tie_word_embeddings", False),
            declared_dtype=metadata.declared_dtype,
        )

    def to_json(self) -> dict:
        """config.json content that reads back to this configuration."""
        raw = {
            "architectures": [ARCHITECTURE],
            "model_type": MODEL_TYPE,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "attention_bias": self.attention_bias,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "sliding_window": None,
            "use_sliding_window": False,
            "max_window_layers": self.num_hidden_layers,
        }
        if self.declared_dtype is not None:
            raw["torch_dtype"] = self.declared_dtype
        return raw

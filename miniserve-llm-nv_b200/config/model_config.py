"""Typed configuration of the Qwen3 dense decoder, read from its own ``config.json`` keys.

Follows the contract of miniserve/config/model_config.py:59-215: every size is required and
must be an integer (booleans are refused), ``head_dim`` is read and never inferred from
``hidden_size / num_attention_heads``, the float constants must be finite and positive, and
every option the model code does not implement (biases, dropout, scaled or interleaved RoPE,
sliding windows, another activation) is refused with a message that names the key.  Unlike
that contract, untied output embeddings are accepted (``tie_word_embeddings`` false needs
``lm_head.weight`` in the checkpoint).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .registry import UnsupportedModelError


def _integer(data: Mapping[str, Any], key: str) -> int:
    value = data.get(key)
    if not isinstance(value, int) or isinstance(value, bool):
        raise ValueError(f"{key} must be an integer in the model config, got {value!r}")
    if value <= 0:
        raise ValueError(f"{key} must be positive, got {value}")
    return value


def _number(data: Mapping[str, Any], key: str) -> float:
    value = data.get(key)
    if not isinstance(value, (int, float)) or isinstance(value, bool):
        raise ValueError(f"{key} must be numeric in the model config, got {value!r}")
    return float(value)


def _boolean(data: Mapping[str, Any], key: str, default: bool = False) -> bool:
    value = data.get(key, default)
    if not isinstance(value, bool):
        raise ValueError(f"{key} must be boolean in the model config, got {value!r}")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    """Sizes and constants of one Qwen3 dense checkpoint; immutable."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    architecture: str = "Qwen3ForCausalLM"
    model_type: str = "qwen3"
    hidden_act: str = "silu"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen3Config":
        architectures = data.get("architectures") or ()
        if list(architectures) != ["Qwen3ForCausalLM"] or str(data.get("model_type", "")) != "qwen3":
            raise UnsupportedModelError(
                "UNSUPPORTED_MODEL_CONFIGURATION: expected architectures ['Qwen3ForCausalLM'] with model_type "
                f"'qwen3', got {list(architectures)!r} with {data.get('model_type')!r}")
        if "head_dim" not in data:
            raise ValueError("Qwen3 model config must define integer head_dim (it is not hidden_size / heads)")
        config = cls(
            hidden_size=_integer(data, "hidden_size"),
            intermediate_size=_integer(data, "intermediate_size"),
            num_hidden_layers=_integer(data, "num_hidden_layers"),
            num_attention_heads=_integer(data, "num_attention_heads"),
            num_key_value_heads=_integer(data, "num_key_value_heads"),
            head_dim=_integer(data, "head_dim"),
            vocab_size=_integer(data, "vocab_size"),
            max_position_embeddings=_integer(data, "max_position_embeddings"),
            rms_norm_eps=_number(data, "rms_norm_eps"),
            rope_theta=_number(data, "rope_theta"),
            tie_word_embeddings=_boolean(data, "tie_word_embeddings"),
            hidden_act=str(data.get("hidden_act", "")),
        )
        if config.hidden_act != "silu":
            raise ValueError(f"hidden_act must be 'silu' (the only gated activation implemented), got {config.hidden_act!r}")
        if _boolean(data, "attention_bias") or _boolean(data, "mlp_bias"):
            raise ValueError("attention_bias and mlp_bias must be false: only bias-free projections are implemented")
        if "attention_dropout" in data and _number(data, "attention_dropout") != 0.0:
            raise ValueError("attention_dropout must be 0.0")
        if _boolean(data, "rope_interleaved") or data.get("rope_scaling") is not None:
            raise ValueError("rope_scaling must be null and rope_interleaved false: scaled or interleaved RoPE is not implemented")
        if _boolean(data, "use_sliding_window"):
            raise ValueError("use_sliding_window must be false: this architecture is implemented without a window")
        config.validate()
        return config

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2 != 0:
            raise ValueError(f"head_dim {self.head_dim} is odd; the rotation pairs the elements of a head")
        from ..kernels import MAX_HEAD_DIM      # a number, no device work: the largest head the attention kernels take

        if self.head_dim > MAX_HEAD_DIM:
            raise ValueError(f"head_dim {self.head_dim} exceeds {MAX_HEAD_DIM}, the largest head size the attention "
                             "kernels of this engine take")
        for name in ("rms_norm_eps", "rope_theta"):
            value = getattr(self, name)
            if not math.isfinite(value) or value <= 0:
                raise ValueError(f"{name} must be finite and positive, got {value}")

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        return {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "attention_dropout": 0.0,
            "rope_scaling": None,
            "sliding_window": None,
            "use_sliding_window": False,
        }

"""Typed configuration of the Llama dense decoder, read from its config.json keys.

Keys, aliases and defaults follow thinruntime/model_arch.py:112-295 (the reference's
``descriptor_from_hf_config``): kv heads default to the head count, ``head_dim`` to
``hidden_size // num_attention_heads``, ``rms_norm_eps`` to 1e-6, ``rope_theta`` to
10000, ``tie_word_embeddings`` to false, and the rotary scaling is read from
``rope_scaling`` or ``rope_parameters`` with ``rope_type`` or ``type`` naming the
variant (thinruntime/model_arch.py:753-760).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from .base import ConfigError, first_value, optional_int, read_config_json, required_int, text_config

SUPPORTED_ROPE_TYPES = ("default", "llama3")
SUPPORTED_ACTIVATIONS = ("silu", "swish")


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of the rotary encoding.  ``rope_type`` ``default`` means
    none; ``llama3`` divides long wavelengths by ``factor`` with a smooth band
    between ``original / high_freq_factor`` and ``original / low_freq_factor``."""

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @staticmethod
    def from_dict(raw: dict[str, Any] | None, fallback_original: int | None) -> "RopeScaling | None":
        if not raw:
            return None
        kind = raw.get("rope_type") or raw.get("type") or "default"
        if kind not in SUPPORTED_ROPE_TYPES:
            raise ConfigError(
                f"rope_scaling type {kind!r} is not supported; supported: {', '.join(SUPPORTED_ROPE_TYPES)}"
            )
        if kind == "default":
            return None
        missing = [k for k in ("factor", "low_freq_factor", "high_freq_factor") if raw.get(k) is None]
        if missing:
            raise ConfigError(f"rope_scaling of type llama3 is missing {missing}")
        original = raw.get("original_max_position_embeddings", fallback_original)
        if original is None:
            raise ConfigError("rope_scaling of type llama3 needs original_max_position_embeddings")
        scaling = RopeScaling(
            rope_type=kind,
            factor=float(raw["factor"]),
            low_freq_factor=float(raw["low_freq_factor"]),
            high_freq_factor=float(raw["high_freq_factor"]),
            original_max_position_embeddings=int(original),
        )
        if scaling.factor <= 0 or scaling.high_freq_factor == scaling.low_freq_factor:
            raise ConfigError(f"rope_scaling has unusable numbers: {raw}")
        return scaling

    def to_dict(self) -> dict[str, Any]:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass(frozen=True)
class LlamaConfig:
    """Every number of a Llama checkpoint.  No size appears anywhere else in code."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling | None = None
    max_position_embeddings: int | None = None
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    bos_token_id: int | None = None
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    architecture: str = field(default="LlamaForCausalLM")

    # ------------------------------------------------------------------ reading
    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "LlamaConfig":
        raw = text_config(raw)
        hidden = required_int(raw, "hidden_size")
        heads = required_int(raw, "num_attention_heads")
        kv_heads = optional_int(raw, "num_key_value_heads", heads)
        head_dim = optional_int(raw, "head_dim", None)
        if head_dim is None:
            if heads <= 0 or hidden % heads:
                raise ConfigError(
                    f"head_dim is absent and hidden_size {hidden} is not a multiple of num_attention_heads {heads}"
                )
            head_dim = hidden // heads
        rope_parameters = raw.get("rope_parameters") if isinstance(raw.get("rope_parameters"), dict) else {}
        theta = first_value(raw, "rope_theta") or rope_parameters.get("rope_theta") or 10000.0
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        arch = raw.get("architectures") or ["LlamaForCausalLM"]
        config = LlamaConfig(
            vocab_size=required_int(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=required_int(raw, "intermediate_size"),
            num_hidden_layers=required_int(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=int(kv_heads),
            head_dim=int(head_dim),
            rms_norm_eps=float(raw.get("rms_norm_eps") or 1e-6),
            rope_theta=float(theta),
            rope_scaling=RopeScaling.from_dict(
                raw.get("rope_scaling") or raw.get("rope_parameters"),
                raw.get("original_max_position_embeddings"),
            ),
            max_position_embeddings=optional_int(raw, "max_position_embeddings", None),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            mlp_bias=bool(raw.get("mlp_bias", False)),
            hidden_act=str(raw.get("hidden_act") or raw.get("hidden_activation") or "silu"),
            bos_token_id=raw.get("bos_token_id"),
            eos_token_ids=eos_ids,
            torch_dtype=str(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
            architecture=str(arch[0]),
        )
        config.validate()
        return config

    @staticmethod
    def from_path(path: str | Path) -> "LlamaConfig":
        return LlamaConfig.from_dict(read_config_json(path))

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        positive = {
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
        }
        for key, value in positive.items():
            if value <= 0:
                raise ConfigError(f"config.json field {key!r} must be positive, got {value}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for the rotary encoding")
        if self.hidden_act not in SUPPORTED_ACTIVATIONS:
            raise ConfigError(
                f"hidden_act {self.hidden_act!r} is not supported; supported: {', '.join(SUPPORTED_ACTIVATIONS)}"
            )
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        """The config.json that reads back to this configuration."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.max_position_embeddings is not None:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out

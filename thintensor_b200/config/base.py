"""Reading config.json: errors, key aliases, and the small helpers every typed
configuration uses.

The reference resolves each required number through a list of alias keys and raises
``config.json is missing required field ...`` when none is present
(thinruntime/model_arch.py:528-550).  The same aliases are kept here so that a
config.json the reference accepts is accepted here.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot describe a model this library runs."""


ALIASES: dict[str, tuple[str, ...]] = {
    "hidden_size": ("hidden_size", "n_embd", "d_model"),
    "intermediate_size": ("intermediate_size", "ffn_dim", "ffn_hidden_size", "n_inner", "d_ff"),
    "num_hidden_layers": ("num_hidden_layers", "n_layer", "num_layers"),
    "num_attention_heads": ("num_attention_heads", "n_head", "num_heads"),
    "num_key_value_heads": ("num_key_value_heads", "num_kv_heads", "n_head_kv"),
    "vocab_size": ("vocab_size", "n_vocab", "padded_vocab_size"),
}


def first_value(raw: dict[str, Any], *names: str) -> Any:
    """The first of ``names`` that config.json gives a non-null value for."""
    for name in names:
        if raw.get(name) is not None:
            return raw[name]
    return None


def required_int(raw: dict[str, Any], key: str) -> int:
    value = first_value(raw, *ALIASES.get(key, (key,)))
    if value is None:
        raise ConfigError(f"config.json is missing required field {key!r}")
    if isinstance(value, bool) or int(value) != value:
        raise ConfigError(f"config.json field {key!r} must be an integer, got {value!r}")
    return int(value)


def optional_int(raw: dict[str, Any], key: str, default: int | None) -> int | None:
    value = first_value(raw, *ALIASES.get(key, (key,)))
    return default if value is None else int(value)


def text_config(raw: dict[str, Any]) -> dict[str, Any]:
    """Multimodal wrappers keep the decoder's numbers under ``text_config``; the
    outer ``architectures``, ``model_type`` and ``tie_word_embeddings`` win
    (thinruntime/model_arch.py:574-592)."""
    inner = raw.get("text_config")
    if not isinstance(inner, dict):
        return raw
    merged = dict(inner)
    for key in ("architectures", "tie_word_embeddings", "model_type"):
        if key in raw:
            merged[key] = raw[key]
    return merged


def read_config_json(path: str | Path) -> dict[str, Any]:
    """``path`` is a model folder or a config.json file."""
    path = Path(path)
    file = path / "config.json" if path.is_dir() else path
    if not file.is_file():
        raise ConfigError(f"no config.json at {file}")
    try:
        raw = json.loads(file.read_text(encoding="utf-8"))
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{file} is not valid JSON: {exc}") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"{file} must hold a JSON object")
    return raw

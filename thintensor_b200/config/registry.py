"""One registry from an architecture's name to its configuration class and to the
function that describes its model.

The reference finds an architecture by comparing a compacted ``model_type`` or
``architectures[0]`` with alias substrings (thinruntime/architectures.py:385-399,
thinruntime/model_arch.py:666-696).  Here ``architectures[0]`` is looked up exactly,
and the compacted ``model_type`` is the fallback.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .base import ConfigError, read_config_json, text_config


@dataclass(frozen=True)
class Architecture:
    name: str                                   # config.json "architectures"[0]
    model_types: tuple[str, ...]                # compacted config.json "model_type" values
    config_class: Any                           # has from_dict(raw) and to_dict()
    describe: Callable[[Any], Any]              # typed configuration -> parts.spec.ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    if arch.name in _ARCHITECTURES:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def supported_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def _compact(value: str) -> str:
    return value.lower().replace("-", "").replace("_", "")


def resolve_architecture(raw: dict[str, Any]) -> Architecture:
    """The registered architecture that a config.json (as a dict) names."""
    _load_builtin()
    raw = text_config(raw)
    names = raw.get("architectures") or []
    if names and names[0] in _ARCHITECTURES:
        return _ARCHITECTURES[names[0]]
    model_type = _compact(str(raw.get("model_type") or ""))
    if model_type:
        for arch in _ARCHITECTURES.values():
            if model_type in arch.model_types:
                return arch
    named = names[0] if names else raw.get("model_type")
    raise ConfigError(
        f"architecture {named!r} is not supported; supported: {', '.join(sorted(_ARCHITECTURES))}"
    )


def load_config(path_or_dict) -> tuple[Architecture, Any]:
    """(architecture, typed configuration) of a model folder, a config.json file or
    an already parsed dict."""
    raw = path_or_dict if isinstance(path_or_dict, dict) else read_config_json(path_or_dict)
    arch = resolve_architecture(raw)
    return arch, arch.config_class.from_dict(raw)


_loaded = False


def _load_builtin() -> None:
    global _loaded
    if not _loaded:
        _loaded = True
        from .. import models  # noqa: F401  (registers the built-in architectures)

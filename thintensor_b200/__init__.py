"""thintensor_b200: a small model library with generation of its own for one NVIDIA
B200, after the dense-decoder engine of random-unknown-username/Thintensor.

Public names are loaded on first use, as the reference does
(thinruntime/__init__.py:14-39), so importing the package is cheap and needs no GPU.
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_EXPORTS = {
    "load_model": ("thintensor_b200.runtime", "load_model"),
    "save_random_model": ("thintensor_b200.runtime", "save_random_model"),
    "random_model": ("thintensor_b200.runtime", "random_model"),
    "Runtime": ("thintensor_b200.runtime", "Runtime"),
    "Engine": ("thintensor_b200.engine.engine", "Engine"),
    "Entry": ("thintensor_b200.engine.engine", "Entry"),
    "DecoderModel": ("thintensor_b200.engine.model", "DecoderModel"),
    "run_generation": ("thintensor_b200.engine.generate", "run_generation"),
    "SamplingParams": ("thintensor_b200.sampling.sampler", "SamplingParams"),
    "SequenceCache": ("thintensor_b200.cache.cache", "SequenceCache"),
    "LlamaConfig": ("thintensor_b200.config.llama", "LlamaConfig"),
    "load_config": ("thintensor_b200.config.registry", "load_config"),
    "register_architecture": ("thintensor_b200.config.registry", "register_architecture"),
    "ModelSpec": ("thintensor_b200.parts.spec", "ModelSpec"),
    "LayerSpec": ("thintensor_b200.parts.spec", "LayerSpec"),
    "PartSpec": ("thintensor_b200.parts.spec", "PartSpec"),
    "Run": ("thintensor_b200.parts.spec", "Run"),
}

__all__ = sorted(_EXPORTS)


def __getattr__(name: str):
    if name in _EXPORTS:
        module, attribute = _EXPORTS[name]
        value = getattr(importlib.import_module(module), attribute)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

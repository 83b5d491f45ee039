"""Random weights from a configuration and a seed, written as a model folder.

The reference has no such mode; its tiny fixtures are freshly initialised library
models saved as bfloat16 safetensors (benchmark_results/operator_graph_matrix.md:5-10).
Here every declared tensor is drawn on the CPU from one generator seeded with ``seed``,
in declaration order: matrices and tables N(0, 0.02), norm weights 1 + N(0, 0.1).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..parts.base import WeightDecl
from .safetensors_io import write_safetensors

STORED_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def draw(decl: WeightDecl, generator: torch.Generator) -> torch.Tensor:
    if decl.integer:
        return torch.zeros(decl.shape, dtype=torch.int32)
    if decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=torch.float32)
    noise = torch.randn(decl.shape, generator=generator, dtype=torch.float32)
    if decl.init == "norm":
        return 1.0 + 0.1 * noise
    if decl.init == "normal":
        return 0.02 * noise
    raise ValueError(f"unknown initialisation {decl.init!r}")


def random_tensors(declared: dict[str, WeightDecl], seed: int, dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    """name -> CPU tensor for every declared tensor that is stored under its own name
    (a tensor that always aliases another one is not drawn)."""
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    out: dict[str, torch.Tensor] = {}
    for name, decl in declared.items():
        if decl.alias_of is not None and decl.prefer_alias:
            continue
        tensor = draw(decl, generator)
        out[name] = tensor.to(dtype) if tensor.is_floating_point() else tensor
    return out


def write_model_folder(folder: str | Path, config, declared: dict[str, WeightDecl], seed: int, dtype: str = "bfloat16") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed
    configuration with ``to_dict``) with weights drawn from ``seed``."""
    if dtype not in STORED_DTYPES:
        raise ValueError(f"weights are stored as bfloat16 or float32, not {dtype!r}")
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = dtype
    (folder / "config.json").write_text(json.dumps(raw, indent=2) + "\n", encoding="utf-8")
    write_safetensors(folder / "model.safetensors", random_tensors(declared, seed, STORED_DTYPES[dtype]),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder

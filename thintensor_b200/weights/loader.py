"""Binding a checkpoint to a model by tensor name.

The model declares what it needs (name, shape); the checkpoint is compared with that
list before anything is copied, and every difference is reported in ONE error: missing
tensors, tensors nobody asked for, and tensors of the wrong shape.  The reference
reports the same classes of fault one at a time (``required layer tensor ... missing``
src/convert_hf.rs:1907-1913, ``layer N missing roles`` thinruntime/execution_plan.py:93-98,
shape and byte checks thinruntime/torch_loader.py:99-113) and only warns about extra
tensors (src/convert_hf.rs:1670-1723).

A checkpoint of a multimodal wrapper (config.json keeps the decoder's numbers under
``text_config``) stores the decoder as ``model.language_model.*`` or ``language_model.*``;
those names are read without the prefix and everything outside it (the other towers)
is left alone, as the reference's converter does (src/convert_hf.rs:613-675, Python
mirror thinruntime/model_arch.py:595-655).  Its renumbering of layers around
cross-attention layers belongs to another architecture and is not done here.

dtype rule: a bfloat16 engine keeps bfloat16 tensors as they are, narrows float16 to
bfloat16 and leaves a tensor that the checkpoint stores in 32-bit floating point in
32 bits; a float32 engine widens every floating tensor to float32.  Integer tables
become int32.
"""
from __future__ import annotations

import fnmatch
from pathlib import Path

import torch

from ..parts.base import WeightDecl
from .safetensors_io import Checkpoint, WeightError

# stored by some exporters, never used: the rotary tables are recomputed
# (the reference lists it as allowed-missing at thinruntime/hf_loader.py:20-25)
IGNORED_PATTERNS = ("*.rotary_emb.inv_freq",)


WRAPPER_PREFIXES = ("model.language_model.", "language_model.")


def decoder_names(stored: list[str]) -> dict[str, str]:
    """Decoder name -> stored name for a wrapper's checkpoint: the prefix goes, ``model.`` is put
    in front of what is not the head and lacks it, tensors outside the prefix are not listed."""
    out: dict[str, str] = {}
    for name in stored:
        suffix = next((name[len(prefix):] for prefix in WRAPPER_PREFIXES if name.startswith(prefix)), None)
        if suffix is None:
            continue
        plain = suffix if suffix == "lm_head.weight" or suffix.startswith("lm_head.") or suffix.startswith("model.") else "model." + suffix
        if plain in out:
            raise WeightError(f"tensors {out[plain]!r} and {name!r} both stand for {plain!r}")
        out[plain] = name
    return out


def compare(declared: dict[str, WeightDecl], stored: dict[str, tuple[int, ...]]) -> tuple[list[str], list[str], list[str]]:
    """(missing, unexpected, wrong_shape) between what a model declares and what a
    checkpoint stores (name -> shape)."""
    missing, wrong = [], []
    used: set[str] = set()
    for name, decl in declared.items():
        source = name
        if decl.alias_of is not None and (decl.prefer_alias or name not in stored):
            source = decl.alias_of
            if name in stored:
                used.add(name)          # a stored copy of a tied tensor is ignored, not unexpected
        if source not in stored:
            if not decl.optional:
                missing.append(name)
            continue
        used.add(source)
        if tuple(stored[source]) != tuple(decl.shape):
            wrong.append(f"{source}: checkpoint has {list(stored[source])}, the model needs {list(decl.shape)}")
    unexpected = [
        name for name in stored
        if name not in used and not any(fnmatch.fnmatch(name, pattern) for pattern in IGNORED_PATTERNS)
    ]
    return missing, unexpected, wrong


def check(declared: dict[str, WeightDecl], stored: dict[str, tuple[int, ...]], where: str) -> None:
    missing, unexpected, wrong = compare(declared, stored)
    if not (missing or unexpected or wrong):
        return
    lines = [f"the checkpoint at {where} does not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
    raise WeightError("\n".join(lines))


def target_dtype(stored: torch.dtype, engine: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_checkpoint(folder: str | Path, declared: dict[str, WeightDecl], engine_dtype: torch.dtype,
                    device: torch.device | str, wrapped: bool = False) -> dict[str, torch.Tensor]:
    """name -> device tensor for every declared tensor the checkpoint (or its alias)
    provides.  An aliased tensor is returned once, under its source's name.  ``wrapped``: the
    folder is a multimodal wrapper's, whose decoder tensors carry a prefix."""
    checkpoint = Checkpoint(folder)
    try:
        stored_as = decoder_names(list(checkpoint.entries)) if wrapped else {name: name for name in checkpoint.entries}
        stored = {name: checkpoint.entries[real].shape for name, real in stored_as.items()}
        check(declared, stored, str(folder))
        out: dict[str, torch.Tensor] = {}
        for name, decl in declared.items():
            source = name
            if decl.alias_of is not None and (decl.prefer_alias or name not in stored):
                source = decl.alias_of
            if source not in stored or source in out:
                continue
            host = checkpoint.tensor(stored_as[source])
            out[source] = host.to(device=device, dtype=target_dtype(host.dtype, engine_dtype)).contiguous()
        return out
    finally:
        checkpoint.close()

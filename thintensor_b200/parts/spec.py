"""The description of a model as data.

An architecture turns its typed configuration into a :class:`ModelSpec`: which parts
each layer is made of, with every size and constant as a parameter, under which
checkpoint names their tensors are stored, and in which order the layers run.  The
engine builds and runs any ModelSpec; it never looks at an architecture's name.

The reference keeps the same information as per-layer ``roles`` and operator names
(thinruntime/execution_plan.py:62-133, thinruntime/operator_registry.py:73-149).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` names a class in the part registry of its role, ``params``
    are that class's constructor arguments (sizes, eps, theta, window ...), and
    ``prefix`` is put before the part's own tensor names to get checkpoint names."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (how the parts are wired around the residual
    stream) and the parts by role.  The ``pre_norm`` arrangement has the roles
    ``mixer_norm``, ``mixer``, ``ffn_norm`` and ``ffn``."""

    arrangement: str
    parts: Mapping[str, PartSpec]


@dataclass(frozen=True)
class Run:
    """One entry of the schedule: run layer ``layer``.  Every run has a cache and a
    state of its own unless ``cache_from`` names an earlier entry of the schedule,
    whose cache this run then reads without writing to it."""

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[Run, ...]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        for index, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule entry {index} names layer {run.layer}, but there are {len(self.layers)} layers")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < index:
                    raise ValueError(f"schedule entry {index} reads the cache of entry {run.cache_from}, which does not run before it")
                if self.schedule[run.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {index} reads the cache of entry {run.cache_from}, which has none of its own")

"""Interfaces of the parts a layer is made of, and one registry for each role.

A part is built from the parameters of its :class:`~thintensor_b200.parts.spec.PartSpec`
alone.  It declares the tensors it needs under names of its own, is handed those
tensors once, and is then run with a :class:`~thintensor_b200.engine.context.StepContext`.
No part knows which model it is in, which layer it is, or what the checkpoint calls
its tensors.

Roles and what each must provide:

* ``Norm``: ``forward(ctx, residual, delta, out, rows=None)`` adds ``delta`` (the not
  yet added output of the part before it, possibly several partial sums) into the
  float32 residual stream and writes the normalised rows to ``out``.
* ``PositionEncoding``: an object a mixer is given at construction.  Its ``kind`` says how
  positions enter the mixer (``"rotary"``: queries and keys are rotated, the mixer's kernels
  take the table that ``rotary()`` returns; ``"none"``); a mixer refuses kinds it cannot apply.
* ``Mixer``: ``forward(ctx, x, cache, states) -> Delta``; declares with ``cache_need()`` /
  ``state_needs()`` what the cache must hold for it: keys and values, and any number of
  per-sequence state tensors of fixed size, each with a shape and dtype of its own.
* ``FeedForward``: ``forward(ctx, x) -> Delta``.
* ``Embedding``: ``forward(ctx, tokens, residual)``; ``Head``: ``forward(ctx, x) -> logits``.
* ``Arrangement``: wires norms, mixer and feed-forward around the residual stream.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class WeightDecl:
    """A tensor a part needs.  ``init`` tells the random-weights mode how to draw it:
    ``normal`` is N(0, 0.02), ``norm`` is 1 + N(0, 0.1), ``zeros`` is zero.
    ``alias_of`` names a checkpoint tensor (full name) to use instead when this one is
    absent from the checkpoint; with ``prefer_alias`` it is used even when this one is
    stored (a tied output head, whose stored copy is ignored)."""

    shape: tuple[int, ...]
    init: str = "normal"
    optional: bool = False
    alias_of: str | None = None
    prefer_alias: bool = False
    integer: bool = False


@dataclass(frozen=True)
class KVNeed:
    """Keys and values a mixer wants kept for each sequence: ``kv_heads`` heads of
    ``head_dim`` numbers per token; ``window`` = only the last so many tokens."""

    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size: one tensor of ``shape`` and ``dtype`` for each
    sequence, zero when the sequence starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Delta:
    """What a mixer or feed-forward adds to the residual stream: float32
    ``[splits, tokens, hidden]``; the sum over ``splits`` is the value.  The norm that
    follows does the sum and the addition.  ``tensor`` is None when the part has already
    added its result into the stream itself (``ctx.residual``, where the arrangement offers it)."""

    tensor: torch.Tensor | None

    @property
    def splits(self) -> int:
        return 0 if self.tensor is None else self.tensor.shape[0]


class Part:
    """Common behaviour: declared weights and binding."""

    def weights(self) -> dict[str, WeightDecl]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """Receive the declared tensors (already on ``device``, in their stored dtype
        unless the engine runs in float32, ``dtype`` being the activation dtype) and
        prepare what kernels need."""

    def projections(self) -> list:
        """The part's weight matrices as :class:`~thintensor_b200.parts.linear.Linear` objects, each
        listed once and each multiplied with every token once per step: what the byte and FLOP
        models of the benchmarks count.  A view of another projection's rows is not listed."""
        return []

    def vectors(self) -> list[torch.Tensor]:
        """Other tensors a step reads once whatever its tokens (a norm's weight)."""
        return []

    def device_driven(self) -> bool:
        """Whether ``forward`` takes everything that changes from step to step from device memory
        (``ctx.tokens``, ``ctx.cu``, ``ctx.len_before``, ``ctx.slots``, the block tables) and, for steps
        of one shape (tokens, sequences, table width, wanted rows), launches the same kernels with
        the same host-side arguments.  Such a step can be captured in a CUDA graph once and
        replayed; a part that looks at ``ctx.host_slots`` / ``host_new`` / ``host_before`` or
        computes on the host must say no.  The engine replays only if every part says yes."""
        return False


class Norm(Part):
    def forward(self, ctx, residual: torch.Tensor, delta: Delta | None, out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
        raise NotImplementedError


@dataclass(frozen=True)
class RotaryTable:
    """What a kernel needs to rotate queries and keys: ``inv_freq`` float32 ``[rotary_dim / 2]`` on
    the device (the angle of pair i at position p is ``p * inv_freq[i]``), ``rotary_dim`` numbers at
    the front of each head are rotated (0: none), cosine and sine are multiplied by
    ``attention_scaling``.  ``signature`` identifies the table's contents."""

    inv_freq: torch.Tensor
    rotary_dim: int
    attention_scaling: float = 1.0
    signature: int = 0      # equal for tables with equal numbers (0: unknown): layers with equal tables can share what a step derives from them


class PositionEncoding(Part):
    """``kind`` is one of ``"rotary"`` and ``"none"``.  A rotary encoding implements ``rotary()``
    (valid after ``bind``); other kinds of encoding (learned tables, additive biases) would add a
    kind and the method that goes with it, and the mixers that can apply it would accept the kind."""

    kind: str = "none"

    def rotary(self) -> RotaryTable:
        raise NotImplementedError(f"a position encoding of kind {self.kind!r} has no rotary table")


class Mixer(Part):
    def cache_need(self) -> KVNeed | None:
        return None

    def state_needs(self) -> list[StateNeed]:
        """Per-sequence state tensors of fixed size, zero when a sequence starts; ``forward`` gets
        one tensor ``[slots, *shape]`` for each, in this order."""
        return []

    def forward(self, ctx, x: torch.Tensor, cache, states: list[torch.Tensor]) -> Delta:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x: torch.Tensor) -> Delta:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx, tokens: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Arrangement:
    """How one layer's parts are wired.  ``roles`` lists the part roles it needs and
    the registry each comes from; ``run`` returns the delta still to be added."""

    roles: dict[str, str] = {}

    def __init__(self, parts: dict[str, Part]):
        self.parts = parts

    def mixers(self) -> list[Mixer]:
        """The layer's mixers (a layer with an attention and a recurrent branch side by side has
        two); each gets a cache and states of its own."""
        return []

    def run(self, ctx, residual: torch.Tensor, pending: Delta | None, caches: list, states: list[list[torch.Tensor]]) -> Delta | None:
        """``caches[i]`` and ``states[i]`` belong to ``mixers()[i]``."""
        raise NotImplementedError

    def device_driven(self) -> bool:
        """See :meth:`Part.device_driven`: an arrangement answers for itself and its parts."""
        return False


class Registry:
    """kind -> class, for one role."""

    def __init__(self, role: str):
        self.role = role
        self._classes: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str):
        def decorate(cls):
            if kind in self._classes:
                raise ValueError(f"{self.role} {kind!r} is already registered")
            self._classes[kind] = cls
            return cls

        return decorate

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def build(self, kind: str, params: dict[str, Any]):
        if kind not in self._classes:
            raise KeyError(f"no {self.role} of kind {kind!r}; registered: {', '.join(sorted(self._classes))}")
        return self._classes[kind](**params)

    def kinds(self) -> list[str]:
        return sorted(self._classes)


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
ARRANGEMENTS = Registry("arrangement")

REGISTRIES = {
    "norm": NORMS,
    "position": POSITION_ENCODINGS,
    "mixer": MIXERS,
    "ffn": FEED_FORWARDS,
    "embedding": EMBEDDINGS,
    "head": HEADS,
    "arrangement": ARRANGEMENTS,
}

"""Rotary position encoding: the table of inverse frequencies a mixer's kernels use.

Default: ``inv_freq[i] = theta ** (-2i / rotary_dim)`` in float32
(thinruntime/gpu_runtime.py:8759-8772).  ``llama3`` scaling: the reference passes the
parameters to a library function (thinruntime/gpu_runtime.py:8779-8816); the rule is
the published one of Llama 3.1: a frequency whose wavelength is shorter than
``original / high_freq_factor`` is kept, one longer than ``original / low_freq_factor``
is divided by ``factor``, and in between the two are blended linearly in
``original / wavelength``.  The angle ``inv_freq * position`` is formed in float32 inside
the kernel; the rotation uses the halves convention (thinruntime/gpu_runtime.py:8703-8712).
"""
from __future__ import annotations

import math

import torch

from .base import POSITION_ENCODINGS, PositionEncoding, RotaryTable


def llama3_scale(inv_freq: torch.Tensor, factor: float, low_freq_factor: float, high_freq_factor: float, original: int) -> torch.Tensor:
    wavelength = 2.0 * math.pi / inv_freq
    smooth = (original / wavelength - low_freq_factor) / (high_freq_factor - low_freq_factor)
    blended = (1.0 - smooth) * inv_freq / factor + smooth * inv_freq
    scaled = torch.where(wavelength > original / low_freq_factor, inv_freq / factor, blended)
    return torch.where(wavelength < original / high_freq_factor, inv_freq, scaled)


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    """``rotary_dim`` numbers at the front of each head are rotated (all of them by
    default); ``scaling`` is None or a dict with ``rope_type`` and that type's numbers."""

    kind = "rotary"

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None, scaling: dict | None = None,
                 attention_scaling: float = 1.0):
        self.head_dim = int(head_dim)
        self.rotary_dim = self.head_dim if rotary_dim is None else int(rotary_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim must be even and within (0, head_dim]; got {self.rotary_dim} for head_dim {self.head_dim}")
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self.attention_scaling = float(attention_scaling)
        self.inv_freq_host = self._table()
        self._rotary: RotaryTable | None = None

    def _table(self) -> torch.Tensor:
        index = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        inv_freq = self.theta ** (-index / self.rotary_dim)
        kind = (self.scaling or {}).get("rope_type", "default")
        if kind == "default":
            return inv_freq
        if kind == "llama3":
            s = self.scaling
            return llama3_scale(inv_freq, float(s["factor"]), float(s["low_freq_factor"]), float(s["high_freq_factor"]),
                                int(s["original_max_position_embeddings"])).to(torch.float32)
        raise ValueError(f"rotary scaling of type {kind!r} is not implemented")

    def bind(self, tensors, dtype, device) -> None:
        signature = hash((self.inv_freq_host.numpy().tobytes(), self.rotary_dim)) or 1
        self._rotary = RotaryTable(self.inv_freq_host.to(device), self.rotary_dim, self.attention_scaling, signature)

    def rotary(self) -> RotaryTable:
        if self._rotary is None:
            raise RuntimeError("the rotary table exists once the encoding has been bound to a device")
        return self._rotary


@POSITION_ENCODINGS.register("none")
class NoEncoding(PositionEncoding):
    """No position encoding: queries and keys go to the cache as projected."""

    kind = "none"

    def __init__(self, head_dim: int):
        self.head_dim = int(head_dim)

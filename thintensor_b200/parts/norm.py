"""RMSNorm over the hidden dimension, fused with the residual addition before it.

``y = x * rsqrt(mean(x^2) + eps) * (w + weight_offset)`` with the statistics in float32
(thinruntime/gpu_runtime.py:13028-13039; the fused add form is the reference's
_add_rms_norm_kernel, thinruntime/triton_kernels.py:2580-2614).  ``weight_offset`` is 0
for Llama (thinruntime/model_arch.py:231-233).
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import NORMS, Delta, Norm, WeightDecl


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, dim: int, eps: float, weight_offset: float = 0.0):
        self.dim = int(dim)
        self.eps = float(eps)
        self.weight_offset = float(weight_offset)
        self.weight: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {"weight": WeightDecl((self.dim,), init="norm")}

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def vectors(self) -> list[torch.Tensor]:
        return [self.weight]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, residual, delta: Delta | None, out, rows=None) -> None:
        api.add_rmsnorm(residual, None if delta is None else delta.tensor, self.weight, self.eps, out, rows, self.weight_offset)   # an empty delta is already in the stream

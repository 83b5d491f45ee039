"""A weight matrix ``[out_features, in_features]`` and the product ``x @ W.T``.

The result is always float32 partial sums ``[splits, tokens, out_features]`` whose sum
over ``splits`` is the product: the kernel that consumes it (the norm that adds it to
the residual stream, the rotary/append kernel, SwiGLU) does that sum, so a projection
whose few output tiles could not fill the GPU may cut its ``in_features`` into slices
without a reduction kernel of its own.

Which kernel runs is decided by the operands alone: bfloat16 activations with a
bfloat16 weight whose rows TMA can address (k a multiple of 8) use the tcgen05
tensor-core kernel; everything else (the true 32-bit path, a weight that the checkpoint
stores in float32, an odd k) uses the exact FMA kernel.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import Delta


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        if weight.dim() != 2:
            raise ValueError(f"a projection weight must be a matrix, got shape {tuple(weight.shape)}")
        self.weight = weight.contiguous()
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        self.out_features, self.in_features = self.weight.shape

    def rows(self, begin: int, end: int) -> "Linear":
        """The projection onto output features begin..end-1 (shares storage)."""
        return Linear(self.weight[begin:end], None if self.bias is None else self.bias[begin:end])

    def __call__(self, ctx, x: torch.Tensor, name: str, into: torch.Tensor | None = None) -> torch.Tensor:
        """``into``: a float32 ``[tokens, out_features]`` tensor of the caller's that receives the
        product itself where k is not cut into slices (the result is then a view of it);
        otherwise the result lies in scratch memory that the next step reuses."""
        tokens = x.shape[0]
        if x.shape[1] != self.in_features:
            raise ValueError(f"{name}: input has {x.shape[1]} features, the weight takes {self.in_features}")
        if into is not None and (into.dtype != torch.float32 or tuple(into.shape) != (tokens, self.out_features) or not into.is_contiguous()):
            raise ValueError(f"{name}: the given output must be contiguous float32 [{tokens}, {self.out_features}]")
        api.set_label(name)
        if api.gemm_tcgen05_usable(x, self.weight):
            splits = api.gemm_tcgen05_splits(tokens, self.out_features, self.in_features)
            if splits == 1 and into is not None:
                out = into.unsqueeze(0)
            else:
                out = ctx.scratch(name, (splits, tokens, self.out_features), torch.float32)
            api.gemm_tcgen05(x, self.weight, self.bias, out, ctx.status, operands_checked=True, shares=self.shares(ctx, tokens))
            return out
        out = into.unsqueeze(0) if into is not None else ctx.scratch(name, (1, tokens, self.out_features), torch.float32)
        api.gemm_simt(x, self.weight, self.bias, out)
        return out


    @staticmethod
    def shares(ctx, tokens: int):
        """Scratch memory for prompts on CTA pairs, whose tiles' k the pairs may share among themselves (one buffer
        for all products of the step: a product is done with it when the next one starts)."""
        if tokens < api.PAIR_TOKENS:
            return None
        return ctx.workspace.get_zeroed("gemm.shares", (api.gemm_tcgen05_shares_words(),), torch.int32)

    def delta(self, ctx, x: torch.Tensor, name: str) -> Delta:
        """The product as an addition to the residual stream.  Where the step offers the stream
        (``ctx.residual``) and the tensor-core kernel can add into its output at no cost of its own
        (prompts whose k is not cut into slices), the product is added there at once and the delta is
        empty; otherwise the delta holds the product's k-slices."""
        residual = getattr(ctx, "residual", None)
        if (residual is not None and residual.shape == (x.shape[0], self.out_features) and api.gemm_tcgen05_usable(x, self.weight)
                and api.gemm_tcgen05_accumulate_pays(x.shape[0], self.out_features, self.in_features)):
            api.set_label(name)
            api.gemm_tcgen05(x, self.weight, self.bias, residual.unsqueeze(0), ctx.status, operands_checked=True, accumulate=True,
                             shares=self.shares(ctx, x.shape[0]))
            return Delta(None)
        return Delta(self(ctx, x, name))


class GatedLinear:
    """gate and up projections as one ``[2 * inter, in]`` matrix (gate rows first) and
    ``silu(gate) * up`` in the activation dtype."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, gate_bias: torch.Tensor | None, up_bias: torch.Tensor | None):
        self.inter = gate.shape[0]
        bias = None
        if gate_bias is not None or up_bias is not None:
            zeros = torch.zeros(self.inter, dtype=torch.float32, device=gate.device)
            bias = torch.cat([(gate_bias if gate_bias is not None else zeros).float(), (up_bias if up_bias is not None else zeros).float()])
        self.fused = Linear(torch.cat([gate, up], dim=0), bias)

    def __call__(self, ctx, x: torch.Tensor, name: str) -> torch.Tensor:
        tokens = x.shape[0]
        act = ctx.scratch(name + ".act", (tokens, self.inter))
        w = self.fused
        if w.bias is None and api.gemm_tcgen05_usable(x, w.weight) and (
                tokens > api.SKINNY_TOKENS or api.gemm_tcgen05_splits(tokens, 2 * self.inter, x.shape[1]) == 1):
            # the float32 gate/up never reach global memory.  With few tokens this form cannot cut k
            # into slices, so it is taken only where the plain product would not slice either
            # (measured on a B200: 3 % faster for 14336 x 4096 at 8 tokens, 2 % slower for 8192 x 2048).
            api.set_label(name)
            api.gemm_tcgen05_swiglu(x, w.weight, act, ctx.status)
            return act
        api.swiglu(w(ctx, x, name), act)
        return act

"""Token embedding and output head.

``h0 = E[token] * scale`` with scale 1 for Llama (thinruntime/gpu_runtime.py:10072,
thinruntime/model_arch.py:234-238).  The head is ``lm_head.weight`` when the checkpoint
has one and the embedding table otherwise (thinruntime/gpu_runtime.py:10395-10401);
logits are float32.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import EMBEDDINGS, HEADS, Embedding, Head, WeightDecl
from .linear import Linear


@EMBEDDINGS.register("table")
class TokenEmbedding(Embedding):
    def __init__(self, vocab: int, hidden: int, scale: float = 1.0):
        self.vocab, self.hidden, self.scale = int(vocab), int(hidden), float(scale)
        self.table: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {"weight": WeightDecl((self.vocab, self.hidden))}

    def bind(self, tensors, dtype, device) -> None:
        self.table = tensors["weight"].contiguous()

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, tokens, residual) -> None:
        api.embed_gather(self.table, tokens, residual, self.scale, ctx.status)


@HEADS.register("linear")
class LinearHead(Head):
    """``fallback`` is the checkpoint name of the tensor that serves as the head when
    the checkpoint stores none (the embedding table); with ``tied`` it is used even if
    a head is stored."""

    def __init__(self, hidden: int, vocab: int, fallback: str | None = None, tied: bool = False, bias: bool = False):
        self.hidden, self.vocab, self.fallback, self.tied, self.bias = int(hidden), int(vocab), fallback, bool(tied), bool(bias)
        self.linear: Linear | None = None

    def weights(self) -> dict[str, WeightDecl]:
        out = {"weight": WeightDecl((self.vocab, self.hidden), alias_of=self.fallback, prefer_alias=self.tied)}
        if self.bias:
            out["bias"] = WeightDecl((self.vocab,))
        return out

    def bind(self, tensors, dtype, device) -> None:
        self.linear = Linear(tensors["weight"], tensors.get("bias"))

    def projections(self) -> list:
        return [self.linear]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x) -> torch.Tensor:
        """Float32 logits ``[rows, vocab]``: in ``ctx.logits_out`` where the step gave one and the
        product could write there, else in scratch memory."""
        into = ctx.logits_out if ctx.logits_out is not None and ctx.logits_out.shape[0] == x.shape[0] else None
        logits = self.linear(ctx, x, "head.logits", into)
        if logits.shape[0] == 1:
            return logits[0]
        return logits.sum(dim=0)

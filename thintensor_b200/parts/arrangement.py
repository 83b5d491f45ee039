"""How a layer's parts are wired around the residual stream.

``pre_norm``: ``h += mixer(norm(h)); h += ffn(norm(h))``, the order of
thinruntime/gpu_runtime.py:10114-10390.  The residual stream is float32; a part's
output is handed on as a :class:`Delta` and added by the next norm's kernel, so the
layer's second addition is done by the following layer's first norm (or by the final
norm).
"""
from __future__ import annotations

from .base import ARRANGEMENTS, Arrangement, Delta


@ARRANGEMENTS.register("pre_norm")
class PreNorm(Arrangement):
    roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "ffn"}

    def mixer(self):
        return self.parts["mixer"]

    def run(self, ctx, residual, pending: Delta | None, cache, state) -> Delta:
        hidden = residual.shape[-1]
        normed = ctx.scratch("block.normed", (ctx.n_tokens, hidden))
        self.parts["mixer_norm"].forward(ctx, residual, pending, normed)
        mixed = self.parts["mixer"].forward(ctx, normed, cache, state)
        self.parts["ffn_norm"].forward(ctx, residual, mixed, normed)
        return self.parts["ffn"].forward(ctx, normed)

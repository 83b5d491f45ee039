"""How a layer's parts are wired around the residual stream.

``pre_norm``: ``h += mixer(norm(h)); h += ffn(norm(h))``, the order of
thinruntime/gpu_runtime.py:10114-10390.  The residual stream is float32; a part's
output is handed on as a :class:`Delta` and added by the next norm's kernel, so the
layer's second addition is done by the following layer's first norm (or by the final
norm).  For long prompts the output projections add their product into the stream themselves
(their tensor-core kernel's epilogue reads and writes the tile once, which spares the
norm kernel a read of the product and a write of the stream); the delta is then empty.
"""
from __future__ import annotations

from .base import ARRANGEMENTS, Arrangement, Delta


@ARRANGEMENTS.register("pre_norm")
class PreNorm(Arrangement):
    roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "ffn"}

    def mixers(self):
        return [self.parts["mixer"]]

    def device_driven(self) -> bool:
        return all(part.device_driven() for part in self.parts.values())

    def run(self, ctx, residual, pending: Delta | None, caches, states) -> Delta:
        hidden = residual.shape[-1]
        # Between a part's output and the norm that follows nothing else reads the stream, so a part
        # may add its output into it directly instead of handing it on.
        ctx.residual = residual
        normed = ctx.scratch("block.normed", (ctx.n_tokens, hidden))
        self.parts["mixer_norm"].forward(ctx, residual, pending, normed)
        mixed = self.parts["mixer"].forward(ctx, normed, caches[0], states[0])
        self.parts["ffn_norm"].forward(ctx, residual, mixed, normed)
        return self.parts["ffn"].forward(ctx, normed)

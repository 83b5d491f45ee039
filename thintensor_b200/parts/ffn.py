"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))`` with
``silu(g) = g / (1 + exp(-g))`` (thinruntime/gpu_runtime.py:10286-10366; the activation
at :10351 and thinruntime/triton_kernels.py:2760-2774)."""
from __future__ import annotations

from .base import FEED_FORWARDS, Delta, FeedForward, WeightDecl
from .linear import GatedLinear, Linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden: int, inter: int, bias: bool = False):
        self.hidden, self.inter, self.bias = int(hidden), int(inter), bool(bias)
        self.gate_up: GatedLinear | None = None
        self.down: Linear | None = None

    def weights(self) -> dict[str, WeightDecl]:
        out = {
            "gate_proj.weight": WeightDecl((self.inter, self.hidden)),
            "up_proj.weight": WeightDecl((self.inter, self.hidden)),
            "down_proj.weight": WeightDecl((self.hidden, self.inter)),
        }
        if self.bias:
            out.update({"gate_proj.bias": WeightDecl((self.inter,)), "up_proj.bias": WeightDecl((self.inter,)),
                        "down_proj.bias": WeightDecl((self.hidden,))})
        return out

    def bind(self, tensors, dtype, device) -> None:
        self.gate_up = GatedLinear(tensors["gate_proj.weight"], tensors["up_proj.weight"],
                                   tensors.get("gate_proj.bias"), tensors.get("up_proj.bias"))
        self.down = Linear(tensors["down_proj.weight"], tensors.get("down_proj.bias"))

    def projections(self) -> list:
        return [self.gate_up.fused, self.down]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x) -> Delta:
        act = self.gate_up(ctx, x, "ffn.gate_up")
        return self.down.delta(ctx, act, "ffn.down")

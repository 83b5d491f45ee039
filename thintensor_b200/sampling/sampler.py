"""Choosing the next token from float32 logits.

The reference's runtime is greedy only (``argmax`` of the float logits,
thinruntime/gpu_runtime.py:11204; its command line rejects anything else,
thinruntime/cli.py:1940-1945).  Its stress script samples on the host with
temperature, top-k and top-p (scripts/stress_validate_thin.py:831-856); the same
distribution is sampled here on the device: scores = logits / temperature, scores
below the k-th largest dropped, then tokens dropped once the probability of all
larger ones exceeds top_p, softmax of the rest, inverse CDF in token-id order.  The
uniform number is a function of (seed, request, step) only, so what a request draws
does not depend on the batch it runs in.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import api


@dataclass(frozen=True)
class SamplingParams:
    """``temperature`` 0 is greedy (lowest id on ties); ``top_k`` 0 and ``top_p`` 1
    switch those filters off, as on the reference's command line
    (thinruntime/cli.py:178-184)."""

    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


def sample(logits: torch.Tensor, params: SamplingParams, request: torch.Tensor, step: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = the token chosen from logits[i]; ``request`` and ``step`` (int32 per
    row) select the uniform number of each row when sampling."""
    if params.greedy:
        api.argmax_rows(logits, out)
    else:
        api.sample_rows(logits, params.temperature, params.top_k, params.top_p, params.seed, request, step, out)

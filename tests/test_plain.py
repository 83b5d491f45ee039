"""The plain implementation itself: against the reference runtime's own logits
(tests/golden/reference_logits.npz, made by tests/golden/make_golden.py), and against
properties that follow from the formulas."""
from __future__ import annotations

import math
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden  # noqa: E402


def golden_config(c: dict) -> dict:
    return {"vocab": c["vocab"], "hidden": c["hidden"], "inter": c["inter"], "layers": c["layers"], "heads": c["heads"],
            "kv_heads": c["kv_heads"], "head_dim": c["head_dim"], "eps": c["eps"], "theta": c["theta"], "scaling": c["scaling"],
            "tied": c["tied"]}


@pytest.mark.parametrize("name", ["a", "b", "f"])
def test_plain_matches_reference_runtime(name):
    """Same weights, same tokens: the reference's CPU runtime (token by token through its
    cache) and the plain implementation (whole sequence, no cache) give the same logits."""
    golden = np.load(GOLDEN / "reference_logits.npz")
    c = make_golden.CONFIGS[name]
    weights = {k: v.double() for k, v in make_golden.golden_weights(c).items()}
    for index, (length, seed) in enumerate(make_golden.PROMPTS[name]):
        tokens = make_golden.prompt_tokens(c["vocab"], length, seed)
        got = plain_llama.forward(golden_config(c), weights, tokens)[-8:]
        want = torch.from_numpy(golden[f"{name}_{index}"]).double()
        assert got.shape == want.shape
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 2e-5 * scale, f"tiny {name} prompt {index}"
        assert bool((got.argmax(-1) == want.argmax(-1)).all())


def test_llama3_frequencies_have_three_bands():
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    plain = plain_llama.rope_inv_freq(32, 500000.0, None)
    scaled = plain_llama.rope_inv_freq(32, 500000.0, scaling)
    ratio = (scaled / plain).tolist()
    assert ratio[0] == 1.0 and ratio[1] == 1.0                   # short wavelengths are kept
    assert 1.0 / 8.0 < ratio[2] < 1.0                            # the band in between is blended
    assert all(abs(r - 1.0 / 8.0) < 1e-6 for r in ratio[3:])     # long wavelengths are divided by the factor
    # the values the reference's runtime reported for this configuration
    np.testing.assert_allclose(scaled[:4].numpy(), [1.0, 0.44036663, 0.07940301, 0.01067464], rtol=2e-6)


def test_rope_is_a_rotation_by_position_difference():
    inv_freq = plain_llama.rope_inv_freq(16, 10000.0, None)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 16, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, 16, generator=g, dtype=torch.float64)

    def score(pq, pk):
        cq = plain_llama.rope_cos_sin(inv_freq, torch.tensor([pq]), torch.float64)
        ck = plain_llama.rope_cos_sin(inv_freq, torch.tensor([pk]), torch.float64)
        return float((plain_llama.apply_rope(q, *cq) * plain_llama.apply_rope(k, *ck)).sum())

    assert abs(score(7, 3) - score(14, 10)) < 1e-6
    assert abs(float(plain_llama.apply_rope(q, *plain_llama.rope_cos_sin(inv_freq, torch.tensor([5]), torch.float64)).norm()) - float(q.norm())) < 1e-9


def test_attention_is_causal_and_grouped():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(6, 4, 8, generator=g, dtype=torch.float64)
    k = torch.randn(6, 2, 8, generator=g, dtype=torch.float64)
    v = torch.randn(6, 2, 8, generator=g, dtype=torch.float64)
    out = plain_llama.causal_attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 0.0, 100.0                                  # the future must not matter
    assert torch.equal(plain_llama.causal_attention(q, k2, v2)[:4], out[:4])
    assert torch.allclose(out[0].reshape(4, 8), v[0].repeat_interleave(2, dim=0))   # position 0 sees itself only; heads 0,1 -> kv 0
    windowed = plain_llama.causal_attention(q, k, v, window=2)
    assert torch.allclose(windowed[:2], out[:2]) and not torch.allclose(windowed[5], out[5])


def test_rms_norm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    want = x / math.sqrt(12.5 + 1e-6) * w
    assert torch.allclose(plain_llama.rms_norm(x, w, 1e-6), want)
    weights = {"gate_proj.weight": torch.eye(2, dtype=torch.float64), "up_proj.weight": 2 * torch.eye(2, dtype=torch.float64),
               "down_proj.weight": torch.eye(2, dtype=torch.float64)}
    got = plain_llama.swiglu(x, weights, "")
    assert torch.allclose(got, x / (1 + torch.exp(-x)) * 2 * x)


def test_sampling_probabilities_and_uniforms():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 2.0])
    p = plain_llama.sampling_probabilities(logits, 1.0, top_k=2)
    assert p[1] == 0 and p[2] == 0 and abs(float(p[0]) - 0.5) < 1e-12     # ties with the k-th stay
    p = plain_llama.sampling_probabilities(torch.tensor([3.0, 1.0, 0.0]), 1.0, top_p=0.5)
    assert p.tolist() == [1.0, 0.0, 0.0]                                   # the first token already exceeds 0.5
    p = plain_llama.sampling_probabilities(torch.tensor([1.0, 1.0, 1.0, -5.0]), 1.0, top_p=0.7)
    assert float(p[3]) == 0.0 and float(p[:3].sum()) == pytest.approx(1.0)
    assert plain_llama.select_token(torch.tensor([1.0, 5.0, 5.0]), 0.0, 0, 1.0, 0, 0, 0) == 1   # greedy: lowest id on ties
    us = [plain_llama.uniform(4, r, s) for r in range(20) for s in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 990
    assert abs(sum(us) / len(us) - 0.5) < 0.03
    assert plain_llama.uniform(4, 3, 7) == plain_llama.uniform(4, 3, 7) != plain_llama.uniform(5, 3, 7)

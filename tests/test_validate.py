"""`validate`'s judge from outside the engine: reading reference logits in both accepted forms, and
the measures and tiers (no GPU)."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

from thintensor_b200.validate import ReferenceLogitsError, comparison_record, load_reference_logits, tier_of


def test_reference_logits_from_npz_and_from_a_trace_folder(tmp_path):
    logits = np.random.default_rng(0).random((10, 7))
    np.savez(tmp_path / "a.npz", tokens=np.arange(10), positions=np.array([1, 5]), logits=logits[[1, 5]])
    tokens, positions, rows = load_reference_logits(tmp_path / "a.npz", 7)
    assert tokens == list(range(10)) and positions == [1, 5] and rows.shape == (2, 7)
    np.savez(tmp_path / "b.npz", logits=logits)
    tokens, positions, rows = load_reference_logits(tmp_path / "b.npz", 7)
    assert tokens is None and positions == list(range(10))
    with pytest.raises(ReferenceLogitsError, match="vocabulary is 8"):
        load_reference_logits(tmp_path / "b.npz", 8)
    np.savez(tmp_path / "c.npz", other=logits)
    with pytest.raises(ReferenceLogitsError, match="no array named 'logits'"):
        load_reference_logits(tmp_path / "c.npz", 7)

    trace = tmp_path / "trace"
    trace.mkdir()
    with pytest.raises(ReferenceLogitsError, match="no trace.jsonl"):
        load_reference_logits(trace, 7)
    steps = [{"step": 0, "entries": [{"id": "y", "tokens": [1, 2, 3], "want": [2]}, {"id": "x", "tokens": [0, 1, 2, 3, 4, 5], "want": [0, 5]}], "end": ["y"]},
             {"step": 3, "entries": [{"id": "x", "tokens": [6, 7], "want": []}], "end": []},
             {"step": 4, "entries": [{"id": "x", "tokens": [8, 9], "want": [1]}], "end": ["x"]}]
    (trace / "trace.jsonl").write_text("".join(json.dumps(s) + "\n" for s in steps))
    np.concatenate([np.zeros((1, 7)), logits[[0, 5]]]).astype("<f4").tofile(trace / "0.f32")
    logits[[9]].astype("<f4").tofile(trace / "4.f32")
    tokens, positions, rows = load_reference_logits(trace, 7, "x")
    assert tokens == list(range(10)) and positions == [0, 5, 9]
    assert np.allclose(rows.numpy(), logits[[0, 5, 9]].astype("float32"))
    tokens, positions, rows = load_reference_logits(trace, 7)             # the trace's first request
    assert tokens == [1, 2, 3] and positions == [2]
    (trace / "4.f32").unlink()
    with pytest.raises(ReferenceLogitsError, match="4.f32 is missing"):
        load_reference_logits(trace, 7, "x")


def test_tiers():
    want = torch.randn(6, 50, generator=torch.Generator().manual_seed(1)) * 3
    same = comparison_record(want + 1e-6, want)
    assert same["top1_same"] and same["top5_ordered_same"] and tier_of([same]) == "exact_pass"
    shifted = comparison_record(want.roll(1, dims=0), want)
    assert tier_of([same, shifted]) == "fail"
    # a swap among near-equal top candidates is a tie within the error of the comparison, not a failure
    close = want.clone()
    top = close.topk(2, dim=-1).indices
    close[0, top[0, 0]], close[0, top[0, 1]] = 100.0, 100.0 - 1e-5
    other = close.clone()
    other[0, top[0, 0]], other[0, top[0, 1]] = 100.0 - 2e-5, 100.0
    record = comparison_record(other, close)
    assert not record["top1_same"] and record["top1_same_or_tied"] and tier_of([record]) == "ranking_pass"

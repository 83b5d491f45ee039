"""``validate``: the engine's ways of running compared with its own true 32-bit path.

One token sequence is run (1) whole in one step, (2) with its last 32 tokens one per
step, (3) together with two shorter sequences in one batch; each in the requested dtype,
and compared position by position with the float32 engine run whole.  The measures and
tiers are the reference's (scripts/compare_hf_thin_logits.py:1890-1967 and :2017-2048):
top-1 equality, ordered top-5, top-5 overlap, cosine, largest and mean absolute error;
``exact_pass`` needs top-1, ordered top-5 and cosine >= 0.999 everywhere, ``ranking_pass``
top-1 and cosine >= 0.99, anything else is ``fail``.  One rule is this library's own: a
top-1 difference does not count when the two candidates are closer in the 32-bit logits
than twice the largest error at that position (a tie within the error of the comparison,
which random weights with their tiny logits produce all the time).
"""
from __future__ import annotations

import torch

from .engine.engine import Entry
from .runtime import load_model


def comparison_record(got: torch.Tensor, want: torch.Tensor) -> dict:
    got, want = got.double(), want.double()
    diff = (got - want).abs()
    top_got, top_want = got.topk(5, dim=-1).indices, want.topk(5, dim=-1).indices
    overlap = [len(set(a.tolist()) & set(b.tolist())) / 5.0 for a, b in zip(top_got, top_want)]
    picked = want.gather(1, top_got[:, :1])[:, 0]                  # the 32-bit logit of the other run's choice
    tied = (want.max(dim=-1).values - picked) <= 2.0 * diff.max(dim=-1).values
    return {
        "positions": got.shape[0],
        "top1_same": bool((top_got[:, 0] == top_want[:, 0]).all()),
        "top1_same_or_tied": bool(((top_got[:, 0] == top_want[:, 0]) | tied).all()),
        "top5_ordered_same": bool((top_got == top_want).all()),
        "top5_overlap": min(overlap),
        "cosine_similarity": float(torch.nn.functional.cosine_similarity(got, want, dim=-1).min()),
        "max_abs_logit_error": float(diff.max()),
        "mean_abs_logit_error": float(diff.mean()),
    }


def tier_of(records: list[dict]) -> str:
    if all(r["top1_same"] and r["top5_ordered_same"] and r["cosine_similarity"] >= 0.999 for r in records):
        return "exact_pass"
    if all(r["top1_same_or_tied"] and r["cosine_similarity"] >= 0.99 for r in records):
        return "ranking_pass"
    return "fail"


def _whole(runtime, tokens):
    engine = runtime.new_engine(max_tokens=len(tokens) + 64, max_sequences=1)
    slot = engine.open()
    logits = engine.step([Entry(slot, tokens, list(range(len(tokens))))]).clone()
    engine.close(slot)
    engine.check_status()
    return logits


def _tail_by_one(runtime, tokens, tail=32):
    tail = min(tail, len(tokens) - 1)
    head = len(tokens) - tail
    engine = runtime.new_engine(max_tokens=len(tokens) + 64, max_sequences=1)
    slot = engine.open()
    got = [engine.step([Entry(slot, tokens[:head], list(range(head)))]).clone()]
    for t in range(head, len(tokens)):
        got.append(engine.step([Entry(slot, [tokens[t]], [0])]).clone())
    engine.close(slot)
    engine.check_status()
    return torch.cat(got)


def _batched(runtime, tokens):
    others = [tokens[: max(1, len(tokens) // 3)], tokens[: max(1, len(tokens) // 7)]]
    engine = runtime.new_engine(max_tokens=3 * (len(tokens) + 64), max_sequences=3)
    slots = [engine.open() for _ in range(3)]
    entries = [Entry(slots[0], others[0], []), Entry(slots[1], tokens, list(range(len(tokens)))), Entry(slots[2], others[1], [])]
    logits = engine.step(entries).clone()
    for slot in slots:
        engine.close(slot)
    engine.check_status()
    return logits


def validate_model(folder, dtype="bf16", tokens=None, length=96, seed=0, device="cuda") -> dict:
    exact = load_model(folder, dtype="fp32", device=device)
    if tokens is None:
        g = torch.Generator().manual_seed(seed)
        tokens = torch.randint(0, exact.model.spec.vocab_size, (length,), generator=g).tolist()
    want = _whole(exact, tokens)
    runtime = exact if dtype in ("fp32", "float32") else load_model(folder, dtype=dtype, device=device)
    records = {}
    for name, run in (("whole", _whole), ("tail_by_one", _tail_by_one), ("unequal_batch", _batched)):
        records[name] = comparison_record(run(runtime, tokens), want)
    return {"model": str(folder), "dtype": str(dtype), "tokens": len(tokens), "against": "float32 engine, whole sequence",
            "modes": records, "tier": tier_of(list(records.values()))}

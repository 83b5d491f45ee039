"""``validate``: the engine's ways of running compared with logits from outside it.

One token sequence is run (1) whole in one step, (2) with its last 32 tokens one per
step, (3) together with two shorter sequences in one batch; each in the requested dtype,
and compared position by position with reference logits.  The reference is a file that
anything may have written (``--reference-logits``): an ``.npz`` with ``logits``
``[n, vocab]``, optionally ``positions`` ``[n]`` (default: the first n) and ``tokens`` (the
sequence they belong to), or a folder of ``<step>.f32`` files as ``bin/trace_run`` writes
them together with the ``trace.jsonl`` that was fed to it; this is the reference's
persisted-logit comparison (scripts/compare_saved_logits.py:35-153).  Without such a file
the judge is the engine's own float32 path run whole, which shows rounding and
batching faults of the bfloat16 path but not a fault both paths share.  The measures and
tiers are the reference's (scripts/compare_hf_thin_logits.py:1890-1967 and :2017-2048):
top-1 equality, ordered top-5, top-5 overlap, cosine, largest and mean absolute error;
``exact_pass`` needs top-1, ordered top-5 and cosine >= 0.999 everywhere, ``ranking_pass``
top-1 and cosine >= 0.99, anything else is ``fail``.  One rule is this library's own: a
top-1 difference does not count when the two candidates are closer in the 32-bit logits
than twice the largest error at that position (a tie within the error of the comparison,
which random weights with their tiny logits produce all the time).
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
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


class ReferenceLogitsError(ValueError):
    pass


def load_reference_logits(path, vocab: int, request: str | None = None):
    """Reference logits from a file somebody else wrote.  Returns ``(tokens or None, positions,
    logits [n, vocab] float64)``: the logits at ``positions`` of the sequence ``tokens``.

    * ``FILE.npz``: ``logits`` [n, vocab]; ``positions`` [n] (default 0..n-1); ``tokens`` (optional).
    * a folder: ``trace.jsonl`` with the steps fed to ``bin/trace_run`` and the ``<step>.f32``
      files it wrote; the logits of one request (``request``, default the trace's first) are
      collected over all steps, by position in that request's token sequence."""
    path = Path(path)
    if path.is_file():
        try:
            data = np.load(path)
        except Exception as exc:  # noqa: BLE001 - any unreadable file is the same error to the user
            raise ReferenceLogitsError(f"{path} is not a readable .npz file: {exc}") from None
        if "logits" not in data:
            raise ReferenceLogitsError(f"{path} holds no array named 'logits' (it has: {', '.join(data.files)})")
        logits = torch.from_numpy(np.asarray(data["logits"], dtype=np.float64))
        if logits.dim() != 2 or logits.shape[1] != vocab:
            raise ReferenceLogitsError(f"reference logits are {tuple(logits.shape)}; the model's vocabulary is {vocab}")
        positions = [int(x) for x in data["positions"]] if "positions" in data else list(range(logits.shape[0]))
        if len(positions) != logits.shape[0]:
            raise ReferenceLogitsError(f"{len(positions)} positions for {logits.shape[0]} rows of logits")
        tokens = [int(t) for t in data["tokens"]] if "tokens" in data else None
        return tokens, positions, logits
    if not path.is_dir():
        raise ReferenceLogitsError(f"{path} is neither a file nor a folder")
    trace = path / "trace.jsonl"
    if not trace.is_file():
        raise ReferenceLogitsError(f"{path} has no trace.jsonl (the steps that produced its .f32 files)")
    tokens: list[int] = []
    found: dict[int, torch.Tensor] = {}
    for line in trace.read_text(encoding="utf-8").splitlines():
        if not line.strip():
            continue
        record = json.loads(line)
        entries = record.get("entries", [])
        if request is None and entries:
            request = str(entries[0]["id"])
        wanted_rows = sum(len(e.get("want", [])) for e in entries)
        rows = None
        row = 0
        for entry in entries:
            want = [int(w) for w in entry.get("want", [])]
            if str(entry["id"]) == request:
                base = len(tokens)
                tokens.extend(int(t) for t in entry["tokens"])
                if want:
                    if rows is None:
                        file = path / f"{record['step']}.f32"
                        if not file.is_file():
                            raise ReferenceLogitsError(f"{file} is missing although step {record['step']} wants logits")
                        rows = torch.from_numpy(np.fromfile(file, dtype="<f4").astype(np.float64))
                        if rows.numel() != wanted_rows * vocab:
                            raise ReferenceLogitsError(f"{file} holds {rows.numel()} numbers, not {wanted_rows} x {vocab}")
                        rows = rows.view(wanted_rows, vocab)
                    for k, place in enumerate(want):
                        found[base + place] = rows[row + k]
            row += len(want)
    if not found:
        raise ReferenceLogitsError(f"the trace in {path} wants no logits of request {request!r}")
    positions = sorted(found)
    return tokens, positions, torch.stack([found[p] for p in positions])


def validate_model(folder, dtype="bf16", tokens=None, length=96, seed=0, device="cuda", reference_logits=None, request=None) -> dict:
    """Run the three modes in ``dtype`` and compare them with ``reference_logits`` (a path, see
    :func:`load_reference_logits`) at the positions that file covers, or, without one, with this
    engine's float32 path at every position."""
    runtime = load_model(folder, dtype=dtype, device=device)
    vocab = runtime.model.spec.vocab_size
    positions = None
    if reference_logits is not None:
        ref_tokens, positions, want = load_reference_logits(reference_logits, vocab, request)
        if ref_tokens is not None:
            if tokens is not None and list(tokens) != ref_tokens:
                raise ReferenceLogitsError("the reference file names other tokens than the ones given")
            tokens = ref_tokens
        against = f"reference logits from {reference_logits}"
    if tokens is None:
        g = torch.Generator().manual_seed(seed)
        tokens = torch.randint(0, vocab, (length,), generator=g).tolist()
    if reference_logits is None:
        exact = runtime if dtype in ("fp32", "float32") else load_model(folder, dtype="fp32", device=device)
        want = _whole(exact, tokens)
        against = "float32 engine, whole sequence (no outside reference given)"
    elif max(positions) >= len(tokens) or min(positions) < 0:
        raise ReferenceLogitsError(f"the reference covers position {max(positions)}, the sequence has {len(tokens)} tokens")
    records = {}
    for name, run in (("whole", _whole), ("tail_by_one", _tail_by_one), ("unequal_batch", _batched)):
        got = run(runtime, tokens)
        if positions is not None:
            got = got[torch.tensor(positions, device=got.device)]
        records[name] = comparison_record(got.cpu(), want.cpu())
    return {"model": str(folder), "dtype": str(dtype), "tokens": len(tokens), "against": against,
            "positions_compared": len(tokens) if positions is None else len(positions),
            "modes": records, "tier": tier_of(list(records.values()))}

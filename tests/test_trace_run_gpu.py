"""bin/trace_run as a user drives it: a subprocess fed JSON lines, logits read back from
the files it writes, compared with the plain implementation.  The same requests are
replayed whole, with the last 32 tokens one by one, and in batches of unequal lengths
that follow one another with a cache that is just large enough."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import ROOT, TINY, assert_close, oracle_logits, token_ids

pytestmark = pytest.mark.gpu


def run_trace(folder: Path, dtype: str, out: Path, max_tokens: int, steps: list[dict]) -> None:
    lines = "".join(json.dumps(s) + "\n" for s in steps)
    done = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(max_tokens)],
        input=lines, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]


def read_step(out: Path, step: int, vocab: int) -> torch.Tensor:
    return torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, vocab).copy())


# a, b: every replay mode in both precisions; d, e (head sizes 64 and 128): the tensor-core attention kernels
@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("a", "bfloat16"), ("b", "float32"), ("b", "bfloat16"),
                                        ("d", "bfloat16"), ("e", "bfloat16")])
def test_replay_modes_agree_with_plain(model_folders, tmp_path, name, dtype):
    folder = model_folders(name, "float32" if dtype == "float32" else "bfloat16")
    vocab = TINY[name]["vocab_size"]
    requests = {f"r{i}": token_ids(vocab, n, 1100 + i) for i, n in enumerate([40, 33, 75, 130, 64])}
    oracle = {k: oracle_logits(folder, v) for k, v in requests.items()}

    # 1. whole, each request alone
    steps = [{"step": i, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}], "end": [k]}
             for i, (k, v) in enumerate(requests.items())]
    run_trace(folder, dtype, tmp_path / "whole", max(-(-len(v) // 64) * 64 for v in requests.values()), steps)
    for i, k in enumerate(requests):
        assert_close(read_step(tmp_path / "whole", i, vocab), oracle[k], dtype, f"whole {k}")

    # 2. the last 32 tokens one by one
    steps, expect, n = [], [], 0
    for k, v in requests.items():
        head = len(v) - 32
        steps.append({"step": n, "entries": [{"id": k, "tokens": v[:head], "want": [head - 1]}], "end": []})
        expect.append((n, k, [head - 1]))
        n += 1
        for t in range(head, len(v)):
            steps.append({"step": n, "entries": [{"id": k, "tokens": [v[t]], "want": [0]}], "end": [k] if t == len(v) - 1 else []})
            expect.append((n, k, [t]))
            n += 1
    run_trace(folder, dtype, tmp_path / "tail", max(-(-len(v) // 64) * 64 for v in requests.values()), steps)
    for step, k, places in expect:
        assert_close(read_step(tmp_path / "tail", step, vocab), oracle[k][places], dtype, f"tail {k} step {step}")

    # 3. batches of unequal lengths: prompts of different lengths start together, then one
    # token each; shorter requests end earlier; the second batch reuses what the first gave back
    batches = [["r0", "r3", "r1"], ["r2", "r4"]]
    prompt_len = {"r0": 7, "r3": 100, "r1": 1, "r2": 64, "r4": 20}
    steps, expect, n = [], [], 0
    for batch in batches:
        at = {k: prompt_len[k] for k in batch}
        steps.append({"step": n, "entries": [{"id": k, "tokens": requests[k][: at[k]], "want": [at[k] - 1]} for k in batch], "end": []})
        expect.append((n, [(k, at[k] - 1) for k in batch]))
        n += 1
        live = list(batch)
        while live:
            entries, wanted, ending = [], [], []
            for k in live:
                entries.append({"id": k, "tokens": [requests[k][at[k]]], "want": [0] if at[k] % 3 else []})
                if at[k] % 3:
                    wanted.append((k, at[k]))
                at[k] += 1
                if at[k] == len(requests[k]):
                    ending.append(k)
            steps.append({"step": n, "entries": entries, "end": ending})
            expect.append((n, wanted))
            n += 1
            live = [k for k in live if k not in ending]
    most = max(sum(-(-len(requests[k]) // 64) * 64 for k in batch) for batch in batches)
    run_trace(folder, dtype, tmp_path / "batched", most, steps)
    for step, wanted in expect:
        if not wanted:
            assert not (tmp_path / "batched" / f"{step}.f32").exists()
            continue
        got = read_step(tmp_path / "batched", step, vocab)
        want = torch.stack([oracle[k][place] for k, place in wanted])
        assert_close(got, want, dtype, f"batched step {step}")

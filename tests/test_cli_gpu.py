"""The command line as a user runs it: random model folder, run, validate, bench."""
from __future__ import annotations

import json
import subprocess
import sys

import pytest

import plain_llama
from conftest import ROOT, TINY

pytestmark = pytest.mark.gpu


def cli(*args, expect=0):
    done = subprocess.run([sys.executable, "-m", "thintensor_b200", *args], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert done.returncode == expect, done.stderr[-2000:]
    return done.stdout


def test_random_run_validate_bench(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY["b"]))
    folder = tmp_path / "model"
    assert cli("random", str(folder), "--config", str(tmp_path / "config.json"), "--seed", "2", "--dtype", "float32").strip() == str(folder)
    out = json.loads(cli("run", str(folder), "--prompt-token-ids", "5,17,3", "--prompt-token-ids", "9", "--max-new-tokens", "6",
                         "--dtype", "fp32", "--ignore-eos", "--json"))
    cfg, weights = plain_llama.read_model(folder)
    assert out["generated_token_ids"] == [plain_llama.generate(cfg, weights, p, 6) for p in ([5, 17, 3], [9])]
    sampled = json.loads(cli("run", str(folder), "--prompt-token-ids", "5,17,3", "--steps", "6", "--temperature", "0.8", "--top-k", "40",
                             "--top-p", "0.9", "--seed", "4", "--dtype", "fp32", "--ignore-eos", "--json"))
    assert sampled["generated_token_ids"] == [plain_llama.generate(cfg, weights, [5, 17, 3], 6, temperature=0.8, top_k=40, top_p=0.9, seed=4)]
    report = json.loads(cli("validate", str(folder), "--dtype", "bf16", "--length", "80", "--json"))
    assert report["tier"] in ("exact_pass", "ranking_pass") and set(report["modes"]) == {"whole", "tail_by_one", "unequal_batch"}
    bench = json.loads(cli("bench", str(folder), "--steps", "8", "--warmup", "3", "--prompt-len", "20", "--batch", "2", "--json"))
    assert bench["tokens_per_s"] > 0 and bench["prefill_tokens_per_s"] > 0 and bench["batch_size"] == 2
    shaped = json.loads(cli("bench", "--shape", "tiny-a", "--steps", "6", "--warmup", "3", "--prompt-len", "9", "--batch", "1,3", "--json"))
    assert [b["batch_size"] for b in shaped["batches"]] == [1, 3] and all(b["tokens_per_s"] > 0 for b in shaped["batches"])
    cli("bench", expect=1)                                  # neither a folder nor a shape
    # the context limit is checked before anything runs, as the reference does
    cli("run", str(folder), "--prompt-token-ids", "1,2,3", "--max-new-tokens", "10", "--context", "8", expect=2)

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
    assert "no outside reference" in report["against"]
    bench = json.loads(cli("bench", str(folder), "--steps", "8", "--warmup", "3", "--prompt-len", "20", "--batch", "2", "--json"))
    assert bench["tokens_per_s"] > 0 and bench["prefill_tokens_per_s"] > 0 and bench["batch_size"] == 2
    run = bench["batches"][0]
    assert run["bytes_per_step"] > 449_184 * 2 and run["prefill_flops"] > 0 and 0 < run["decode_frac_of_hbm_peak"] < 1.5
    assert 0 < run["prefill_frac_of_tensor_peak"] < 1.5 and bench["peaks"]["source"] in ("measured", "fallback")
    unequal = json.loads(cli("bench", str(folder), "--warmup", "3", "--prompt-len", "5:60", "--batch", "4", "--context", "96", "--to-context",
                             "--profile-classes", "--json"))["batches"][0]
    assert len(unequal["prompt_tokens"]) == 4 and len(set(unequal["prompt_tokens"])) > 1
    assert unequal["steps"] == 96 - max(unequal["prompt_tokens"]) - 3 - 1
    classes = unequal["classes"]
    assert any(k.startswith("tt_gemm") and "ffn.down" in k for k in classes["decode_step"]) and "tt_embed_gather" in classes["prefill_step"]
    assert sum(c["calls"] for c in classes["decode_step"].values()) == unequal["launches_per_step"] or classes["decode_ms_serialised"] > 0
    shaped = json.loads(cli("bench", "--shape", "tiny-a", "--steps", "6", "--warmup", "3", "--prompt-len", "9", "--batch", "1,3", "--json"))
    assert [b["batch_size"] for b in shaped["batches"]] == [1, 3] and all(b["tokens_per_s"] > 0 for b in shaped["batches"])
    cli("bench", expect=1)                                  # neither a folder nor a shape
    # the context limit is checked before anything runs, as the reference does
    cli("run", str(folder), "--prompt-token-ids", "1,2,3", "--max-new-tokens", "10", "--context", "8", expect=2)


def test_validate_against_logits_from_outside(tmp_path):
    """`validate --reference-logits`: the plain implementation's logits as an .npz pass; the same logits
    shifted by a position fail with exit code 1; a folder written in bin/trace_run's format (here by the
    plain implementation) is read through its trace."""
    import numpy as np

    (tmp_path / "config.json").write_text(json.dumps(TINY["a"]))
    folder = tmp_path / "model"
    cli("random", str(folder), "--config", str(tmp_path / "config.json"), "--seed", "5", "--dtype", "float32")
    cfg, weights = plain_llama.read_model(folder)
    tokens = [int(t) for t in np.random.default_rng(3).integers(0, TINY["a"]["vocab_size"], 90)]
    logits = plain_llama.forward(cfg, weights, tokens).numpy()
    positions = list(range(0, 90, 7)) + [88, 89]
    np.savez(tmp_path / "good.npz", tokens=np.array(tokens), positions=np.array(positions), logits=logits[positions])
    for dtype in ("fp32", "bf16"):
        report = json.loads(cli("validate", str(folder), "--dtype", dtype, "--reference-logits", str(tmp_path / "good.npz"), "--json"))
        assert report["tier"] in ("exact_pass", "ranking_pass") and report["positions_compared"] == len(positions)
        assert "good.npz" in report["against"]
    np.savez(tmp_path / "shifted.npz", tokens=np.array(tokens), positions=np.array(positions), logits=logits[[p - 1 for p in positions]])
    report = json.loads(cli("validate", str(folder), "--dtype", "fp32", "--reference-logits", str(tmp_path / "shifted.npz"), "--json", expect=1))
    assert report["tier"] == "fail"
    # the trace_run format: two steps of request "x" (and a bystander), logits of the wanted places per step
    trace = tmp_path / "trace"
    trace.mkdir()
    steps = [{"step": 0, "entries": [{"id": "y", "tokens": [1, 2, 3], "want": [2]}, {"id": "x", "tokens": tokens[:60], "want": [0, 59]}], "end": ["y"]},
             {"step": 1, "entries": [{"id": "x", "tokens": tokens[60:], "want": [0, 29]}], "end": ["x"]}]
    (trace / "trace.jsonl").write_text("".join(json.dumps(s) + "\n" for s in steps))
    other = plain_llama.forward(cfg, weights, [1, 2, 3]).numpy()
    np.concatenate([other[2:3], logits[[0, 59]]]).astype("<f4").tofile(trace / "0.f32")
    logits[[60, 89]].astype("<f4").tofile(trace / "1.f32")
    report = json.loads(cli("validate", str(folder), "--dtype", "fp32", "--reference-logits", str(trace), "--request", "x", "--json"))
    assert report["tier"] == "exact_pass" and report["positions_compared"] == 4

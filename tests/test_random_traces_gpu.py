"""Seeded random traces through the engine against the plain implementation: batches of
random size and random prompt lengths start together, every sequence then goes on one
token at a time to its own random length, logits are asked for at random places, and
batches follow one another in a cache that is only as large as the largest batch needs.
A trace is a different cut of the same requests every time, so any dependence of the
logits on the cut, on the batch or on the place in the cache shows up as a mismatch."""
from __future__ import annotations

import random

import pytest
import torch

from conftest import TINY, assert_close, oracle_logits, token_ids

pytestmark = pytest.mark.gpu


def random_batches(rng: random.Random, n_batches: int):
    batches = []
    for _ in range(n_batches):
        size = rng.choice([1, 1, 2, 3, 4, 5, 8])
        batch = []
        for _ in range(size):
            prompt = rng.choice([1, 2, 3, 7, 31, 63, 64, 65, 129, rng.randint(1, 150), rng.randint(100, 400)])
            total = prompt + rng.choice([0, 0, 1, 2, 5, rng.randint(0, 40)])
            batch.append((prompt, total))
        batches.append(batch)
    return batches


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed", [("a", 1), ("b", 2), ("c", 3), ("b", 4), ("d", 5), ("e", 6), ("d", 7), ("f", 8)])
def test_random_traces(model_folders, name, seed, dtype):
    import thintensor_b200
    from thintensor_b200.engine.engine import Entry

    folder = model_folders(name, "float32" if dtype == "float32" else "bfloat16")
    runtime = thintensor_b200.load_model(folder, dtype=dtype)
    vocab = TINY[name]["vocab_size"]
    rng = random.Random(1000 * seed + (0 if dtype == "float32" else 1))
    batches = random_batches(rng, 6)
    most = max(sum(-(-total // 64) * 64 for _, total in batch) for batch in batches)
    engine = runtime.new_engine(max_tokens=most, max_sequences=max(len(b) for b in batches),
                                max_step_tokens=rng.choice([8192, 100, 33]))
    ident = 0
    for batch in batches:
        requests = []
        for prompt, total in batch:
            ident += 1
            tokens = token_ids(vocab, total, 5000 + 97 * seed + ident)
            requests.append({"tokens": tokens, "prompt": prompt, "total": total, "slot": engine.open(), "got": {}, "at": 0})
        entries = []
        for r in requests:
            want = sorted(set(rng.sample(range(r["prompt"]), k=min(r["prompt"], rng.choice([0, 1, 2, 3])))) | {r["prompt"] - 1})
            if rng.random() < 0.2:
                want = []
            r["want_now"] = want
            entries.append(Entry(r["slot"], r["tokens"][: r["prompt"]], want))
        logits = engine.step(entries)
        row = 0
        for r in requests:
            for place in r["want_now"]:
                r["got"][place] = logits[row]
                row += 1
            r["at"] = r["prompt"]
        assert row == logits.shape[0]
        live = []
        for r in requests:
            if r["at"] >= r["total"]:
                engine.close(r["slot"])
            else:
                live.append(r)
        while live:
            entries, wanted = [], []
            for r in live:
                ask = rng.random() < 0.7
                entries.append(Entry(r["slot"], [r["tokens"][r["at"]]], [0] if ask else []))
                if ask:
                    wanted.append(r)
            logits = engine.step(entries)
            assert logits.shape[0] == len(wanted)
            for row, r in enumerate(wanted):
                r["got"][r["at"]] = logits[row]
            still = []
            for r in live:
                r["at"] += 1
                if r["at"] >= r["total"]:
                    engine.close(r["slot"])
                else:
                    still.append(r)
            live = still
        engine.check_status()
        for index, r in enumerate(requests):
            if not r["got"]:
                continue
            places = sorted(r["got"])
            want = oracle_logits(folder, r["tokens"])[places]
            assert_close(torch.stack([r["got"][p] for p in places]), want, dtype, f"{name} seed {seed} request {index} {r['prompt']}/{r['total']}")
        assert engine.cache.free_blocks == engine.cache.num_blocks
        assert engine.cache.slots.free_count == engine.cache.max_slots

"""The model that the benchmark times, whole: all 16 layers of the Llama-3.2-1B shape with its
128,256-row tied vocabulary in bfloat16, against the plain implementation; and the decode step as
generation runs it (captured in a CUDA graph and replayed, kernels started under the tail of the
ones before them) held to the plain implementation token by token.

The weights are random, with queries and keys scaled so that attention is peaked (a wrong block,
slot or layer then moves the logits far beyond tolerance) and a table large enough for logits of
order one."""
from __future__ import annotations

import pytest
import torch

import plain_llama
from conftest import TINY, assert_close, oracle_logits, token_ids
from test_real_shapes_gpu import write_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def full_1b(tmp_path_factory):
    """The folder, the engine's runtime and the oracle's logits for one 300-token sequence (made once:
    the oracle's pass over 1.2 billion parameters on the CPU is the slow part)."""
    import thintensor_b200

    folder = write_model(tmp_path_factory.mktemp("full") / "llama-1b", "1b", "bfloat16", layers=16, vocab=128256)
    tokens = token_ids(128256, 300, 41)
    cfg, weights = plain_llama.read_model(folder)
    want = plain_llama.forward(cfg, weights, tokens, dtype=torch.float32).double()
    del weights
    runtime = thintensor_b200.load_model(folder, dtype="bf16")
    return folder, runtime, tokens, want


def test_full_model_whole_tail_and_batched(full_1b):
    from thintensor_b200.engine.engine import Entry

    folder, runtime, tokens, want = full_1b
    vocab = 128256
    engine = runtime.new_engine(max_tokens=1024, max_sequences=3)
    # whole, a handful of positions (the head runs on the wanted rows only)
    places = [0, 1, 63, 64, 100, 255, 256, 290, 299]
    slot = engine.open()
    whole = engine.step([Entry(slot, tokens, places)])
    engine.close(slot)
    engine.check_status()
    assert_close(whole, want[places], "bfloat16", "16 layers, whole")
    # the last 32 tokens one by one
    slot = engine.open()
    got = [engine.step([Entry(slot, tokens[:268], [267])])]
    for t in range(268, 300):
        got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
    engine.close(slot)
    engine.check_status()
    assert_close(torch.cat(got), want[267:300], "bfloat16", "16 layers, tail one by one")
    # inside a batch of unequal lengths that start together; the shortest ends first
    others = [token_ids(vocab, 140, 42), token_ids(vocab, 3, 43)]
    a, b, c = engine.open(), engine.open(), engine.open()
    logits = engine.step([Entry(b, others[0][:130], []), Entry(a, tokens[:258], [0, 257]), Entry(c, others[1][:2], [1])])
    rows = {0: logits[0], 257: logits[1]}
    logits = engine.step([Entry(b, [others[0][130]], []), Entry(a, [tokens[258]], [0]), Entry(c, [others[1][2]], [])])
    rows[258] = logits[0]
    engine.close(c)
    for t in range(259, 300):
        logits = engine.step([Entry(a, [tokens[t]], [0]), Entry(b, [others[0][130 + (t - 258) % 10]], [])])
        rows[t] = logits[0]
    engine.close(a)
    engine.close(b)
    engine.check_status()
    order = sorted(rows)
    assert_close(torch.stack([rows[p] for p in order]), want[order], "bfloat16", "16 layers, unequal batch")
    assert engine.cache.free_blocks == engine.cache.num_blocks


def teacher_forced_decode(runtime, prompts, sequences, steps, use_graph):
    """Run the generation loop's decode step (``EngineBackend.decode_step``: tokens fed from the host,
    the step replayed from its CUDA graph when ``use_graph``) with the given sequences' own tokens fed
    in place of the sampled ones, and return each step's logits ``[steps, batch, vocab]``."""
    from thintensor_b200.engine.generate import EngineBackend
    from thintensor_b200.sampling.sampler import SamplingParams

    batch = len(prompts)
    longest = max(len(s) for s in sequences)
    engine = runtime.new_engine(max_tokens=(-(-longest // 64) * 64) * batch, max_sequences=batch)
    backend = EngineBackend(engine, SamplingParams(), use_graph=use_graph)
    backend.start_batch(list(range(batch)), prompts, [len(s) for s in sequences])
    live = list(range(batch))
    out = []
    for step in range(steps):
        backend._last = [sequences[i][len(prompts[i]) + step] for i in range(batch)]       # what the oracle saw at this position
        backend.decode_step(live)
        out.append(backend._state.logits.clone())
    if use_graph:
        assert backend._state.graphs, "the step should have been captured and replayed"
    for position in live:
        backend.finish(position)
    assert engine.cache.free_blocks == engine.cache.num_blocks
    return torch.stack(out)


@pytest.mark.parametrize("name", ["d", "e"])
def test_graph_replayed_decode_against_plain_tiny(model_folders, name):
    """bfloat16 decode steps replayed from a CUDA graph (programmatic dependent launch, weights and
    cache blocks fetched before the wait for the previous kernel) against the plain implementation,
    teacher-forced, for a batch of unequal lengths that crosses block boundaries."""
    import thintensor_b200

    folder = model_folders(name, "bfloat16")
    runtime = thintensor_b200.load_model(folder, dtype="bf16")
    vocab = TINY[name]["vocab_size"]
    steps = 40
    sequences = [token_ids(vocab, n + steps + 1, 300 + n) for n in (50, 7, 121)]
    prompts = [s[: len(s) - steps - 1] for s in sequences]
    got = teacher_forced_decode(runtime, prompts, sequences, steps, use_graph=True)
    for i, sequence in enumerate(sequences):
        want = oracle_logits(folder, sequence)
        first = len(prompts[i])
        assert_close(got[:, i], want[first: first + steps], "bfloat16", f"tiny {name}, graph replay, sequence {i}")


def test_graph_replayed_decode_against_plain_full_model(full_1b):
    """The same at the benchmarked shape: 16 layers, k-sliced few-token products, the fused
    rotation + cache write + attention kernel, the 1,002-CTA head product."""
    folder, runtime, tokens, want = full_1b
    steps = 30
    prompt = tokens[: 300 - steps - 1]
    got = teacher_forced_decode(runtime, [prompt], [tokens], steps, use_graph=True)
    first = len(prompt)
    assert_close(got[:, 0], want[first: first + steps], "bfloat16", "16 layers, graph replay")
    eager = teacher_forced_decode(runtime, [prompt], [tokens], steps, use_graph=False)
    assert torch.equal(got, eager), "replaying the captured step must give the bits of running it"

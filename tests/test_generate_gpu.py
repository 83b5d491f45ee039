"""Generation through the Python entry point against the plain implementation:
greedy tokens, stop tokens, sequences that end earlier, several batches one after
another, sampling with temperature / top-k / top-p, and that graph replay changes nothing."""
from __future__ import annotations

import pytest
import torch

import plain_llama
from conftest import TINY, token_ids

pytestmark = pytest.mark.gpu


def oracle_generate(folder, prompts, max_new, stop_ids=(), **sampling):
    cfg, weights = plain_llama.read_model(folder)
    return [plain_llama.generate(cfg, weights, p, max_new, stop_ids=stop_ids, request=i, **sampling) for i, p in enumerate(prompts)]


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_matches_plain(model_folders, name):
    import thintensor_b200

    folder = model_folders(name, "float32")
    runtime = thintensor_b200.load_model(folder, dtype="fp32")
    vocab = TINY[name]["vocab_size"]
    lengths = [5, 9, 2] if name == "a" else [17, 1, 40, 70]
    prompts = [token_ids(vocab, n, 700 + n) for n in lengths]
    steps = 8 if name == "a" else 12
    got = runtime.generate(prompts, max_new_tokens=steps, stop_ids=(), batch_size=4)
    assert got == oracle_generate(folder, prompts, steps)
    # the same without graph replay, and in smaller batches so that slots are reused
    assert runtime.generate(prompts, max_new_tokens=steps, stop_ids=(), batch_size=2, use_graph=False) == got
    # the per-step path (host reads every token) gives the same tokens as the run without host reads
    assert runtime.generate(prompts, max_new_tokens=steps, stop_ids=(-1,), batch_size=3) == got


def test_stop_tokens_end_sequences_early(model_folders):
    import thintensor_b200
    from thintensor_b200.engine.generate import GenerationStats

    name = "b"
    folder = model_folders(name, "float32")
    runtime = thintensor_b200.load_model(folder, dtype="fp32")
    vocab = TINY[name]["vocab_size"]
    prompts = [token_ids(vocab, n, 800 + n) for n in (6, 30, 3, 11, 19)]
    free_run = oracle_generate(folder, prompts, 24)
    # stop ids taken from what the model actually produces, so that sequences end at different steps
    stop = {free_run[0][3], free_run[1][10], free_run[3][1]}
    want = oracle_generate(folder, prompts, 24, stop_ids=stop)
    assert len({len(w) for w in want}) > 1, "the stop ids should end sequences at different lengths"
    stats = GenerationStats()
    got = runtime.generate(prompts, max_new_tokens=24, stop_ids=tuple(stop), batch_size=3, stats=stats)
    assert got == want
    assert stats.batches == 2 and stats.batch_sizes == [3, 2]
    engine = runtime._engine
    assert engine.cache.free_blocks == engine.cache.num_blocks
    assert engine.cache.slots.free_count == engine.cache.max_slots


def test_an_error_in_a_batch_leaves_the_cache_whole(model_folders):
    """A request that the step refuses (a token outside the vocabulary) ends the call with an
    error; the slots and blocks of its batch are given back, so the next call has the whole cache."""
    import thintensor_b200
    from thintensor_b200.engine.engine import StepError

    folder = model_folders("a", "float32")
    runtime = thintensor_b200.load_model(folder, dtype="fp32")
    vocab = TINY["a"]["vocab_size"]
    prompts = [token_ids(vocab, n, 900 + n) for n in (4, 7, 3)]
    want = runtime.generate(prompts, max_new_tokens=6, stop_ids=(), batch_size=3)
    with pytest.raises(StepError, match="outside the vocabulary"):
        runtime.generate([prompts[0], prompts[1] + [vocab], prompts[2]], max_new_tokens=6, stop_ids=(), batch_size=3)
    cache = runtime._engine.cache
    assert cache.free_blocks == cache.num_blocks and cache.slots.free_count == cache.max_slots
    assert runtime.generate(prompts, max_new_tokens=6, stop_ids=(), batch_size=3) == want


@pytest.mark.parametrize("sampling", [
    {"temperature": 0.8, "seed": 4},
    {"temperature": 1.3, "top_k": 5, "seed": 9},
    {"temperature": 0.7, "top_p": 0.6, "seed": 1},
    {"temperature": 1.0, "top_k": 20, "top_p": 0.9, "seed": 123456789012},
])
def test_sampling_matches_plain(model_folders, sampling):
    """Tiny B with temperature sampling: the same counter-based uniform numbers on both
    sides give the same tokens, whatever the batch a request runs in."""
    import thintensor_b200

    name = "b"
    folder = model_folders(name, "float32")
    runtime = thintensor_b200.load_model(folder, dtype="fp32")
    vocab = TINY[name]["vocab_size"]
    prompts = [token_ids(vocab, n, 900 + n) for n in (17, 1, 40, 70)]
    want = oracle_generate(folder, prompts, 12, **sampling)
    got = runtime.generate(prompts, max_new_tokens=12, stop_ids=(), batch_size=4, **sampling)
    assert got == want
    assert runtime.generate(prompts, max_new_tokens=12, stop_ids=(), batch_size=1, **sampling) == got


def test_bfloat16_greedy_follows_float32(model_folders):
    """bfloat16 generation is the same model: teacher-forced on the float32 tokens its
    argmax agrees wherever the float32 margin is clear."""
    import thintensor_b200
    from thintensor_b200.engine.engine import Entry

    name = "a"
    folder = model_folders(name, "bfloat16")
    exact = thintensor_b200.load_model(folder, dtype="fp32")
    fast = thintensor_b200.load_model(folder, dtype="bf16")
    prompt = token_ids(TINY[name]["vocab_size"], 12, 1000)
    new = exact.generate([prompt], max_new_tokens=20, stop_ids=())[0]
    tokens = prompt + new
    outs = []
    for runtime in (exact, fast):
        engine = runtime.new_engine(max_tokens=128, max_sequences=1)
        slot = engine.open()
        outs.append(engine.step([Entry(slot, tokens, list(range(len(tokens))))]))
        engine.close(slot)
    top2 = outs[0].topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.25
    assert int(clear.sum()) > 5
    assert bool((outs[0].argmax(-1) == outs[1].argmax(-1))[clear].all())


@pytest.mark.parametrize("name,dtype", [("b", "fp32"), ("d", "bf16")])
def test_captured_decode_steps_serve_later_batches(model_folders, name, dtype):
    """The engine keeps the captured decode step of a batch shape.  Later batches of that shape
    (other prompts, other slots and blocks, other lengths inside the same number of blocks) must
    replay it with their own data; a step whose scratch memory has moved since the capture (a
    longer prompt in between) must be captured again; and other sampling parameters must not
    reuse a graph that has the old ones baked in."""
    import thintensor_b200

    folder = model_folders(name, "float32" if dtype == "fp32" else "bfloat16")
    runtime = thintensor_b200.load_model(folder, dtype=dtype)
    fresh = thintensor_b200.load_model(folder, dtype=dtype)
    vocab = TINY[name]["vocab_size"]

    def both(prompts, steps, **kw):
        got = runtime.generate(prompts, max_new_tokens=steps, stop_ids=(-1,), batch_size=len(prompts), context=512, **kw)
        new_engine = fresh.new_engine(max_tokens=512 * len(prompts), max_sequences=len(prompts))
        from thintensor_b200.engine.generate import EngineBackend, run_generation
        from thintensor_b200.sampling.sampler import SamplingParams
        params = SamplingParams(kw.get("temperature", 0.0), kw.get("top_k", 0), kw.get("top_p", 1.0), kw.get("seed", 0))
        want = run_generation(EngineBackend(new_engine, params, use_graph=False), prompts, steps, (-1,), len(prompts), 512, None)
        assert got == want
        return got

    first = [token_ids(vocab, n, 40 + n) for n in (20, 33, 7)]
    both(first, 100)                                                      # 133 tokens at most: three blocks per sequence
    engine = runtime._engine
    states = dict(engine.decode_states)
    assert len(states) == 1
    second = [token_ids(vocab, n, 90 + n) for n in (9, 30, 25)]          # same shape: 3 sequences, three blocks each
    both(second, 100)
    assert runtime._engine is engine and dict(engine.decode_states) == states, "the same shape should reuse the captured step"
    generation = engine.workspace.generation
    both([token_ids(vocab, 180, 5)], 6)                                   # a long prompt on the same engine: scratch memory grows
    assert runtime._engine is engine and engine.workspace.generation > generation
    both(first, 100)                                                      # the old graph holds stale addresses and is replaced
    both(second, 100, temperature=0.9, seed=3)                            # other sampling parameters: another state
    assert len(engine.decode_states) == 3

"""The engine against the plain implementation, under every way of cutting the work:
each request alone and whole; with its last 32 tokens one by one; in batches of unequal
lengths whose shorter requests end earlier, one batch after another so that slots and
blocks are used again; long decoding; the first tokens of a sequence."""
from __future__ import annotations

import pytest
import torch

from conftest import TINY, assert_close, oracle_logits, token_ids

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["a", "b", "c", "d", "e", "f"]


def load(folder, dtype):
    import thintensor_b200

    return thintensor_b200.load_model(folder, dtype=dtype, device="cuda")


def folder_for(model_folders, name, dtype):
    # the bfloat16 engine reads bfloat16 weights; the oracle reads the same file, so
    # both compute with identical weight values
    return model_folders(name, "float32" if dtype == "float32" else "bfloat16")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests_alone(model_folders, name, dtype):
    from thintensor_b200.engine.engine import Entry

    folder = folder_for(model_folders, name, dtype)
    runtime = load(folder, dtype)
    engine = runtime.new_engine(max_tokens=512, max_sequences=4)
    vocab = TINY[name]["vocab_size"]
    for seed, length in enumerate([1, 2, 5, 63, 64, 65, 130, 200]):
        tokens = token_ids(vocab, length, 100 + seed)
        slot = engine.open()
        logits = engine.step([Entry(slot, tokens, list(range(length)))])
        engine.close(slot)
        engine.check_status()
        assert_close(logits, oracle_logits(folder, tokens), dtype, f"{name} whole length {length}")
    assert engine.cache.free_blocks == engine.cache.num_blocks


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_tokens_one_by_one(model_folders, name, dtype):
    from thintensor_b200.engine.engine import Entry

    folder = folder_for(model_folders, name, dtype)
    runtime = load(folder, dtype)
    engine = runtime.new_engine(max_tokens=512, max_sequences=2)
    vocab = TINY[name]["vocab_size"]
    for seed, length in enumerate([33, 70, 161]):
        tokens = token_ids(vocab, length, 200 + seed)
        want = oracle_logits(folder, tokens)
        head = length - 32
        slot = engine.open()
        got = [engine.step([Entry(slot, tokens[:head], [head - 1])])]
        for t in range(head, length):
            got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
        engine.close(slot)
        engine.check_status()
        assert_close(torch.cat(got), want[head - 1:], dtype, f"{name} tail of length {length}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_from_empty_cache(model_folders, name, dtype):
    """Token by token from the very first token: positions 0, 1, 2 ... of a fresh slot."""
    from thintensor_b200.engine.engine import Entry

    folder = folder_for(model_folders, name, dtype)
    runtime = load(folder, dtype)
    engine = runtime.new_engine(max_tokens=128, max_sequences=2)
    tokens = token_ids(TINY[name]["vocab_size"], 20, 300)
    slot = engine.open()
    got = [engine.step([Entry(slot, [t], [0])]) for t in tokens]
    engine.close(slot)
    assert_close(torch.cat(got), oracle_logits(folder, tokens), dtype, f"{name} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_reuse(model_folders, name, dtype):
    """Batches of unequal prompts; every request is then continued one token per step
    to its own length, so shorter requests leave earlier; the next batch reuses the
    slots and blocks.  The cache is sized so that nothing is left over."""
    from thintensor_b200.engine.engine import Entry

    folder = folder_for(model_folders, name, dtype)
    runtime = load(folder, dtype)
    vocab = TINY[name]["vocab_size"]
    # (prompt length, total length) per request
    batches = [
        [(5, 9), (9, 40), (2, 2), (17, 30)],
        [(70, 75), (1, 12), (40, 41)],
        [(64, 70), (3, 67), (128, 131), (31, 33)],
    ]
    most = max(sum(-(-total // 64) * 64 for _, total in batch) for batch in batches)
    engine = runtime.new_engine(max_tokens=most, max_sequences=4)
    seed = 400
    for batch_index, batch in enumerate(batches):
        requests = []
        for prompt_len, total in batch:
            seed += 1
            requests.append({"tokens": token_ids(vocab, total, seed), "prompt": prompt_len, "total": total,
                             "slot": engine.open(), "got": {}})
        logits = engine.step([Entry(r["slot"], r["tokens"][: r["prompt"]], [r["prompt"] - 1]) for r in requests])
        for row, r in enumerate(requests):
            r["got"][r["prompt"] - 1] = logits[row]
            r["at"] = r["prompt"]
        live = [r for r in requests if r["at"] < r["total"]]
        for r in requests:
            if r["at"] >= r["total"]:
                engine.close(r["slot"])
        while live:
            logits = engine.step([Entry(r["slot"], [r["tokens"][r["at"]]], [0]) for r in live])
            for row, r in enumerate(live):
                r["got"][r["at"]] = logits[row]
                r["at"] += 1
            for r in live:
                if r["at"] >= r["total"]:
                    engine.close(r["slot"])
            live = [r for r in live if r["at"] < r["total"]]
        engine.check_status()
        for index, r in enumerate(requests):
            want = oracle_logits(folder, r["tokens"])
            places = sorted(r["got"])
            assert places == list(range(r["prompt"] - 1, r["total"]))
            got = torch.stack([r["got"][p] for p in places])
            assert_close(got, want[places], dtype, f"{name} batch {batch_index} request {index}")
        assert engine.cache.free_blocks == engine.cache.num_blocks
        assert engine.cache.slots.free_count == engine.cache.max_slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model_folders, dtype):
    """Several hundred decode steps after a short prompt: every block boundary and the
    split of the keys over several slices are crossed."""
    from thintensor_b200.engine.engine import Entry

    name = "b"
    folder = folder_for(model_folders, name, dtype)
    runtime = load(folder, dtype)
    engine = runtime.new_engine(max_tokens=1024, max_sequences=2)
    tokens = token_ids(TINY[name]["vocab_size"], 450, 500)
    want = oracle_logits(folder, tokens)
    slot = engine.open()
    got = [engine.step([Entry(slot, tokens[:3], [2])])]
    for t in range(3, len(tokens)):
        got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
    engine.close(slot)
    engine.check_status()
    assert_close(torch.cat(got), want[2:], dtype, "long decoding")


@pytest.mark.parametrize("name", ["d", "e"])
def test_long_context_and_many_sequences_on_the_tensor_core_kernels(model_folders, name):
    """bfloat16 with head sizes 64 and 128.  A prompt of 4,700 tokens (the prompt attention's
    long loop), then decoding over it: the keys are cut into more than 8 slices (scratch and merge
    kernel).  Then 80 short sequences decoded together: more CTAs than SMs, which for head size 64
    is the variant with half the warps; and slices combined by a thread-block cluster in between
    (a 1,300-token context).  A peaked attention makes a lost slice or block show."""
    from thintensor_b200.engine.engine import Entry

    dtype = "bfloat16"
    folder = folder_for(model_folders, name, dtype)
    runtime = load(folder, dtype)
    vocab = TINY[name]["vocab_size"]
    engine = runtime.new_engine(max_tokens=4800 + 80 * 64, max_sequences=81)

    tokens = token_ids(vocab, 4712, 41)
    want = oracle_logits(folder, tokens)
    slot = engine.open()
    head = 4700
    got = [engine.step([Entry(slot, tokens[:head], [0, 1300, head - 1])])]
    for t in range(head, len(tokens)):
        got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
    engine.close(slot)
    engine.check_status()
    assert_close(torch.cat(got), want[[0, 1300] + list(range(head - 1, len(tokens)))], dtype, "long context")

    middle = token_ids(vocab, 1312, 42)
    want = oracle_logits(folder, middle)
    slot = engine.open()
    got = [engine.step([Entry(slot, middle[:1300], [1299])])]
    for t in range(1300, len(middle)):
        got.append(engine.step([Entry(slot, [middle[t]], [0])]))
    engine.close(slot)
    assert_close(torch.cat(got), want[1299:], dtype, "slices combined in a cluster")

    prompts = [token_ids(vocab, 6 + (i * 7) % 50, 900 + i) for i in range(80)]
    slots = [engine.open() for _ in prompts]
    heads = [len(p) - 4 for p in prompts]
    engine.step([Entry(s, p[:h], []) for s, p, h in zip(slots, prompts, heads)])
    check = [0, 17, 42, 79]
    oracle = {i: oracle_logits(folder, prompts[i]) for i in check}
    for t in range(4):
        logits = engine.step([Entry(s, [p[h + t]], [0]) for s, p, h in zip(slots, prompts, heads)])
        for i in check:
            assert_close(logits[i : i + 1], oracle[i][heads[i] + t : heads[i] + t + 1], dtype, f"many sequences, request {i} step {t}")
    for s in slots:
        engine.close(s)
    engine.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_step_cut_into_pieces(model_folders, dtype):
    """A step with more tokens than max_step_tokens runs in pieces with the same result."""
    from thintensor_b200.engine.engine import Entry

    name = "a"
    folder = folder_for(model_folders, name, dtype)
    runtime = load(folder, dtype)
    engine = runtime.new_engine(max_tokens=512, max_sequences=3, max_step_tokens=48)
    vocab = TINY[name]["vocab_size"]
    prompts = [token_ids(vocab, n, 600 + n) for n in (50, 7, 100)]
    slots = [engine.open() for _ in prompts]
    logits = engine.step([Entry(s, p, [0, len(p) - 1]) for s, p in zip(slots, prompts)])
    for s in slots:
        engine.close(s)
    for i, p in enumerate(prompts):
        want = oracle_logits(folder, p)
        assert_close(logits[2 * i: 2 * i + 2], want[[0, len(p) - 1]], dtype, f"pieces request {i}")


def test_bfloat16_engine_keeps_float32_tensors(model_folders):
    """A checkpoint stored in float32 run by the bfloat16 engine: the tensors stay in 32 bits
    (the exact product kernel takes bfloat16 activations with float32 weights), activations and
    cache are bfloat16, and the logits follow the oracle on the float32 weights."""
    import thintensor_b200
    from thintensor_b200.engine.engine import Entry

    name = "c"
    folder = model_folders(name, "float32")
    runtime = thintensor_b200.load_model(folder, dtype="bf16")
    mixer = runtime.model.layers[0].parts["mixer"]
    assert mixer.qkv.weight.dtype == torch.float32 and runtime.model.embedding.part.table.dtype == torch.float32
    engine = runtime.new_engine(max_tokens=256, max_sequences=2)
    assert engine.cache.kv_groups[0].storage.dtype == torch.bfloat16
    tokens = token_ids(TINY[name]["vocab_size"], 90, 700)
    want = oracle_logits(folder, tokens)
    slot = engine.open()
    got = [engine.step([Entry(slot, tokens[:70], list(range(70)))])]
    for t in range(70, 90):
        got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
    engine.close(slot)
    engine.check_status()
    assert_close(torch.cat(got), want, "bfloat16", "float32 checkpoint in the bfloat16 engine")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("d", "bfloat16"), ("e", "bfloat16")])
def test_steps_of_a_known_shape_are_replayed_with_their_own_data(model_folders, name, dtype):
    """The engine captures a step's launches when its shape (tokens, sequences, table width, wanted rows) comes a
    second time and replays them from then on.  Replayed steps must serve other tokens, other slots and blocks, other
    lengths and other wanted places: prompts of one shape for different requests in turn, then decoding token by
    token across a block boundary, all against the plain implementation, with slots freed and reused in between."""
    from thintensor_b200.engine.engine import Entry

    folder = folder_for(model_folders, name, dtype)
    runtime = load(folder, dtype)
    engine = runtime.new_engine(max_tokens=1024, max_sequences=4)
    assert engine.use_step_graphs
    vocab = TINY[name]["vocab_size"]
    # three pairs of prompts with the same packed shape (30 + 50 tokens, one block each, 3 wanted rows) but different cuts
    for round_, (la, lb) in enumerate([(30, 50), (45, 35), (10, 70)]):
        a_tokens, b_tokens = token_ids(vocab, la + 40, 500 + round_), token_ids(vocab, lb + 40, 600 + round_)
        spare = engine.open() if round_ == 1 else None             # shifts the slots and blocks the round gets
        a, b = engine.open(), engine.open()
        logits = engine.step([Entry(a, a_tokens[:la], [0, la - 1]), Entry(b, b_tokens[:lb], [lb // 2])])
        want = torch.cat([oracle_logits(folder, a_tokens)[[0, la - 1]], oracle_logits(folder, b_tokens)[[lb // 2]]])
        assert_close(logits, want, dtype, f"{name} prompts of one shape, round {round_}")
        got_a, got_b = [], []
        for t in range(40):                                         # both cross position 64: the table grows a column, a new shape
            logits = engine.step([Entry(a, [a_tokens[la + t]], [0]), Entry(b, [b_tokens[lb + t]], [0])])
            got_a.append(logits[0])
            got_b.append(logits[1])
        assert_close(torch.stack(got_a), oracle_logits(folder, a_tokens)[la: la + 40], dtype, f"{name} decode a, round {round_}")
        assert_close(torch.stack(got_b), oracle_logits(folder, b_tokens)[lb: lb + 40], dtype, f"{name} decode b, round {round_}")
        for slot in (a, b, spare):
            if slot is not None:
                engine.close(slot)
        engine.check_status()
    assert engine.graph_replays > 100, "prompt rounds 2 and 3 and nearly all decode steps should have been replays"
    assert engine.cache.free_blocks == engine.cache.num_blocks
    # an engine that never replays gives the same prompt logits bit for bit (the same kernels, launched one by one)
    plain = runtime.new_engine(max_tokens=1024, max_sequences=4, step_graphs=False)
    tokens = token_ids(vocab, 80, 700)
    results = []
    for e in (engine, plain, engine):
        slot = e.open()
        results.append(e.step([Entry(slot, tokens, [0, 40, 79])]).clone())
        e.close(slot)
    assert plain.graph_replays == 0
    assert torch.equal(results[0], results[1]) and torch.equal(results[1], results[2])

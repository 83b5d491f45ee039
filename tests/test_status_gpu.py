"""The device status word, which stands in for a memory checker: a kernel that meets a block-table
entry outside the pool, or whose bounded wait runs out, raises a bit, skips the access, and the host
turns the bit into an exception.  Nothing here faults, traps or hangs the GPU: the bad table entry
is met by kernels whose source checks the range before the access, and the wait that runs out is a
bounded one whose limit the test sets to a few milliseconds."""
from __future__ import annotations

import pytest
import torch

from conftest import TINY, assert_close, oracle_logits, token_ids

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_a_wait_that_runs_out_raises_the_status_and_leaves_the_gpu_usable():
    """The tensor-core product's first stage is told to expect bytes that no copy brings, with a wait
    limit of 3 ms: every CTA's waits run out, the kernel returns with STATUS_WAIT_EXPIRED, and the
    same product run normally right after gives the right numbers (tensor memory was given back,
    no copy was left in flight)."""
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(3)
    x = torch.randn(8, 512, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(640, 512, generator=g).to(torch.bfloat16).to(DEV)
    want = x.double() @ w.double().T
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros(2, 8, 640, dtype=torch.float32, device=DEV)
    api.gemm_tcgen05(x, w, None, out, status)                     # compiles, and shows the product is right to begin with
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    torch.testing.assert_close(out.double().sum(0), want, rtol=1e-4, atol=1e-2)
    try:
        api.gemm_tcgen05_failure_drill(wait_limit_ns=3_000_000, undelivered_bytes=1024)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        api.gemm_tcgen05(x, w, None, out, status)
        stop.record()
        torch.cuda.synchronize()                                  # returns: the kernel gave up by itself
        assert start.elapsed_time(stop) < 1000.0, "the waits should have run out within milliseconds"
    finally:
        api.gemm_tcgen05_failure_drill(wait_limit_ns=0, undelivered_bytes=0)
    assert int(status.item()) & api.STATUS_WAIT_EXPIRED
    status.zero_()
    for _ in range(3):                                            # many CTAs allocate tensor memory again on every SM
        out.fill_(float("nan"))
        api.gemm_tcgen05(x, w, None, out, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    torch.testing.assert_close(out.double().sum(0), want, rtol=1e-4, atol=1e-2)


def test_a_wait_that_runs_out_in_decode_attention_raises_the_status_and_leaves_the_gpu_usable():
    """The decode attention streams the cache through mbarriers that count the copies' bytes.  Its warps' first stage is told
    to expect bytes that no copy brings, with a wait limit of 3 ms: every warp's wait runs out, the kernel returns with
    STATUS_WAIT_EXPIRED (the copies themselves have landed, so nothing is in flight when shared memory is given up), and
    the same call run normally right after gives the right numbers."""
    from test_kernels_gpu import attention_reference, make_cache, randn, tol
    from thintensor_b200.kernels import api

    dtype, heads, kv_heads, head_dim = torch.bfloat16, 8, 2, 64
    totals = [300, 70, 1]
    n = len(totals)
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=80)
    q = randn(n, heads, head_dim, dtype=dtype, seed=81)
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    before = torch.tensor([t - 1 for t in totals], dtype=torch.int32, device=DEV)
    scale = head_dim ** -0.5
    want = attention_reference(q.float().cpu(), keys, values, [1] * n, heads, kv_heads, scale, 0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def run():
        out = torch.full((n, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
        api.attention_mma(q.view(n, -1), k_pool, v_pool, table, cu, before, n, n, heads, kv_heads, head_dim, scale, 0, 1, out, None, None,
                          status, one_token_each=True)
        return out

    first = run()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    torch.testing.assert_close(first.double().cpu().view(n, heads, head_dim), want, **tol(dtype))
    try:
        api.attention_mma_failure_drill(wait_limit_ns=3_000_000, undelivered_bytes=256)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run()
        stop.record()
        torch.cuda.synchronize()                                  # returns: the kernel gave up by itself
        assert start.elapsed_time(stop) < 1000.0, "the waits should have run out within milliseconds"
    finally:
        api.attention_mma_failure_drill(wait_limit_ns=0, undelivered_bytes=0)
    assert int(status.item()) & api.STATUS_WAIT_EXPIRED
    status.zero_()
    again = run()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    torch.testing.assert_close(again.double().cpu().view(n, heads, head_dim), want, **tol(dtype))


def test_the_engine_turns_an_expired_wait_into_an_exception(model_folders):
    import thintensor_b200
    from thintensor_b200.engine.engine import Entry
    from thintensor_b200.kernels import api

    folder = model_folders("d", "bfloat16")
    runtime = thintensor_b200.load_model(folder, dtype="bf16")
    engine = runtime.new_engine(max_tokens=256, max_sequences=1)
    tokens = token_ids(TINY["d"]["vocab_size"], 20, 5)
    slot = engine.open()
    engine.step([Entry(slot, tokens[:10], [9])])
    engine.check_status()
    try:
        api.gemm_tcgen05_failure_drill(wait_limit_ns=2_000_000, undelivered_bytes=512)
        engine.step([Entry(slot, tokens[10:11], [0])])
        with pytest.raises(RuntimeError, match="a bounded wait inside a kernel ran out"):
            engine.check_status()
    finally:
        api.gemm_tcgen05_failure_drill(wait_limit_ns=0, undelivered_bytes=0)
    engine.close(slot)
    # the status word was cleared by the check, and the engine serves the next request correctly
    slot = engine.open()
    logits = engine.step([Entry(slot, tokens, list(range(len(tokens))))])
    engine.check_status()
    engine.close(slot)
    assert_close(logits, oracle_logits(folder, tokens), "bfloat16", "after the drill")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("d", "bfloat16"), ("e", "bfloat16")])
def test_a_table_entry_outside_the_pool_is_flagged_and_skipped(model_folders, name, dtype):
    """Two sequences decode together; the first block of one of them is replaced by -1 in its table
    row.  The kernels' own range check skips that block (attention.cu / attention_mma.cu read the entry,
    compare it with the pool size, and only then form an address), STATUS_BAD_BLOCK is raised, and the
    other sequence's logits are what they would have been."""
    import thintensor_b200
    from thintensor_b200.engine.engine import Entry

    folder = model_folders(name, "float32" if dtype == "float32" else "bfloat16")
    runtime = thintensor_b200.load_model(folder, dtype=dtype)
    engine = runtime.new_engine(max_tokens=512, max_sequences=2)
    vocab = TINY[name]["vocab_size"]
    good, bad = token_ids(vocab, 150, 61), token_ids(vocab, 140, 62)
    want = oracle_logits(folder, good)
    a, b = engine.open(), engine.open()
    engine.step([Entry(a, good[:149], []), Entry(b, bad[:139], [])])
    engine.check_status()
    row = engine.cache.kv_groups[0].table.rows[b]
    kept = row[0]
    row[0] = -1                                                     # a block inside the sequence's length that is "gone"
    try:
        logits = engine.step([Entry(a, [good[149]], [0]), Entry(b, [bad[139]], [0])])
        with pytest.raises(RuntimeError, match="a block table entry outside the pool was met"):
            engine.check_status()
    finally:
        row[0] = kept
    assert torch.isfinite(logits).all()
    assert_close(logits[:1], want[149:150], dtype, "the sequence whose table is whole")
    assert not torch.allclose(logits[1].double().cpu(), oracle_logits(folder, bad)[139], atol=1e-3), "the other one lost 64 keys"
    engine.close(a)
    engine.close(b)
    assert engine.cache.free_blocks == engine.cache.num_blocks


def test_generation_with_stop_ids_reports_a_fault_in_the_step_that_had_it(model_folders, monkeypatch):
    """The loop that reads every token on the host (stop ids set) gets the status word with the tokens:
    a fault raises in the step that had it, and the batch's slots and blocks go back to the cache."""
    import thintensor_b200
    from thintensor_b200.engine import generate

    folder = model_folders("a", "float32")
    runtime = thintensor_b200.load_model(folder, dtype="fp32")
    vocab = TINY["a"]["vocab_size"]
    prompts = [token_ids(vocab, n, 70 + n) for n in (70, 9)]
    want = runtime.generate(prompts, max_new_tokens=5, stop_ids=(-1,), batch_size=2)
    original = generate._DecodeState.fill
    calls = {"n": 0}

    def fill_then_lose_a_block(self, *args, **kwargs):
        original(self, *args, **kwargs)
        calls["n"] += 1
        self.tables[0][0, 0] = -1                                   # on the device: the first block of the first sequence

    monkeypatch.setattr(generate._DecodeState, "fill", fill_then_lose_a_block)
    with pytest.raises(RuntimeError, match="a block table entry outside the pool was met"):
        runtime.generate(prompts, max_new_tokens=5, stop_ids=(-1,), batch_size=2)
    assert calls["n"] == 1, "the first decode step should have raised"
    monkeypatch.setattr(generate._DecodeState, "fill", original)
    cache = runtime._engine.cache
    assert cache.free_blocks == cache.num_blocks and cache.slots.free_count == cache.max_slots
    assert runtime.generate(prompts, max_new_tokens=5, stop_ids=(-1,), batch_size=2) == want

"""The generation loop's decisions with a scripted backend: batches, stop tokens,
sequences that end earlier, token limits, and that every sequence is finished exactly once."""
from __future__ import annotations

import pytest

from thintensor_b200.engine.generate import GenerationError, GenerationStats, run_generation
from thintensor_b200.sampling import SamplingParams


class ScriptedBackend:
    """Request r produces script[r][0], script[r][1], ...; records every call."""

    def __init__(self, script, capacity_tokens=10_000, capacity_sequences=100):
        self.script = script
        self.capacity_tokens, self.capacity_sequences = capacity_tokens, capacity_sequences
        self.calls: list[tuple] = []
        self.live_now: set[int] = set()
        self.finished: list[int] = []
        self.batch: list[int] = []
        self.at: dict[int, int] = {}

    def fits(self, totals):
        return sum(totals) + sum(0 for _ in self.live_now) <= self.capacity_tokens and len(totals) <= self.capacity_sequences

    def start_batch(self, requests, prompts, totals):
        assert not self.live_now, "a batch started while the previous one still had live sequences"
        self.calls.append(("start", tuple(requests), tuple(len(p) for p in prompts), tuple(totals)))
        self.batch = list(requests)
        self.live_now = set(range(len(requests)))
        out = []
        for r in requests:
            self.at[r] = 1
            out.append(self.script[r][0])
        return out

    def decode_step(self, live):
        assert set(live) <= self.live_now
        self.calls.append(("step", tuple(live)))
        out = []
        for position in live:
            r = self.batch[position]
            out.append(self.script[r][self.at[r]])
            self.at[r] += 1
        return out

    def decode_run(self, live, steps):
        self.calls.append(("run", tuple(live), steps))
        return [self.decode_step(live) for _ in range(steps)]

    def finish(self, position):
        assert position in self.live_now, "finished twice, or never started"
        self.live_now.remove(position)
        self.finished.append(self.batch[position])

    def abandon(self):
        self.calls.append(("abandon", tuple(sorted(self.live_now))))
        self.live_now.clear()


def test_stop_tokens_and_early_finish():
    script = {0: [5, 6, 99, 1, 1, 1], 1: [99, 2, 2, 2, 2, 2], 2: [7, 7, 7, 7, 7, 7], 3: [8, 99, 0, 0, 0, 0], 4: [4, 4, 4, 99, 0, 0]}
    backend = ScriptedBackend(script)
    stats = GenerationStats()
    out = run_generation(backend, [[1]] * 5, max_new_tokens=5, stop_ids=[99], batch_size=3, stats=stats)
    assert out == [[5, 6, 99], [99], [7, 7, 7, 7, 7], [8, 99], [4, 4, 4, 99]]        # the stop token is kept
    assert sorted(backend.finished) == [0, 1, 2, 3, 4] and not backend.live_now
    steps = [c for c in backend.calls if c[0] == "step"]
    assert steps[:4] == [("step", (0, 2)), ("step", (0, 2)), ("step", (2,)), ("step", (2,))]   # request 1 left after its first token
    assert [c[1] for c in backend.calls if c[0] == "start"] == [(0, 1, 2), (3, 4)]             # no request joins a running batch
    assert stats.batches == 2 and stats.batch_sizes == [3, 2] and stats.new_tokens == 15
    assert stats.decoded_tokens == 15 - 5


def test_without_stop_ids_runs_to_the_limit_without_reading_tokens():
    script = {r: list(range(10)) for r in range(3)}
    backend = ScriptedBackend(script)
    out = run_generation(backend, [[1, 2], [3], [4, 5, 6]], max_new_tokens=6, stop_ids=(), batch_size=8)
    assert out == [list(range(6))] * 3
    assert ("run", (0, 1, 2), 5) in backend.calls and sorted(backend.finished) == [0, 1, 2]
    assert backend.calls[0] == ("start", (0, 1, 2), (2, 1, 3), (8, 7, 9))
    backend = ScriptedBackend(script)
    assert run_generation(backend, [[1]], max_new_tokens=1) == [[0]] and backend.finished == [0]
    assert not [c for c in backend.calls if c[0] in ("run", "step")]


def test_batches_follow_the_cache_capacity():
    script = {r: [1] * 10 for r in range(5)}
    backend = ScriptedBackend(script, capacity_tokens=40)
    prompts = [[0] * 10, [0] * 10, [0] * 30, [0] * 5, [0] * 5]
    run_generation(backend, prompts, max_new_tokens=4, stop_ids=(), batch_size=4)
    assert [c[1] for c in backend.calls if c[0] == "start"] == [(0, 1), (2,), (3, 4)]
    with pytest.raises(GenerationError, match="more than the cache can hold"):
        run_generation(ScriptedBackend(script, capacity_tokens=20), prompts, max_new_tokens=4)


def test_a_failing_step_gives_back_what_the_batch_holds():
    """A backend call that raises in the middle of a batch: the loop frees the batch's unfinished
    sequences before the error goes on, and runs no further batch."""
    script = {0: [5, 99, 0, 0], 1: [6, 6, 6, 6], 2: [7, 7, 7, 7], 3: [8, 8, 8, 8]}

    class Failing(ScriptedBackend):
        def decode_step(self, live):
            if sum(1 for c in self.calls if c[0] == "step") == 2:
                raise RuntimeError("device status 0x4")
            return super().decode_step(live)

    backend = Failing(script)
    with pytest.raises(RuntimeError, match="device status"):
        run_generation(backend, [[1]] * 4, max_new_tokens=4, stop_ids=[99], batch_size=3)
    assert backend.finished == [0]                                  # request 0 had ended on its stop token
    assert backend.calls[-1] == ("abandon", (1, 2)) and not backend.live_now
    assert [c[1] for c in backend.calls if c[0] == "start"] == [(0, 1, 2)]


def test_argument_errors():
    backend = ScriptedBackend({0: [1, 1, 1]})
    with pytest.raises(GenerationError, match="max_new_tokens"):
        run_generation(backend, [[1]], max_new_tokens=0)
    with pytest.raises(GenerationError, match="empty"):
        run_generation(backend, [[]], max_new_tokens=2)
    with pytest.raises(GenerationError, match="exceeds the context"):
        run_generation(backend, [[1] * 10], max_new_tokens=3, context=12)
    with pytest.raises(GenerationError, match="batch_size"):
        run_generation(backend, [[1]], max_new_tokens=2, batch_size=0)
    assert run_generation(backend, [], max_new_tokens=3) == []


def test_sampling_params_are_checked():
    assert SamplingParams().greedy and not SamplingParams(temperature=0.7).greedy
    for bad in ({"temperature": -1.0}, {"top_k": -1}, {"top_p": 0.0}, {"top_p": 1.5}):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_no_cpu_path():
    import thintensor_b200
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(RuntimeError, match="CUDA"):
        thintensor_b200.load_model(".", dtype="bf16", device="cuda")
    with pytest.raises(RuntimeError, match="no CPU path"):
        thintensor_b200.load_model(".", dtype="bf16", device="cpu")


def test_table_widths_fall_into_few_shapes():
    """Decode states are keyed by the width of their block tables: powers of two up to 16
    blocks, then multiples of 16, never less than what the sequences need."""
    from thintensor_b200.engine.generate import table_width

    assert [table_width(b) for b in (0, 1, 2, 3, 4, 5, 8, 9, 16)] == [1, 1, 2, 4, 4, 8, 8, 16, 16]
    assert [table_width(b) for b in (17, 32, 33, 64, 65, 512, 513)] == [32, 32, 48, 64, 80, 512, 528]
    assert all(table_width(b) >= b for b in range(1, 3000))
    assert len({table_width(b) for b in range(1, 1025)}) <= 5 + 63


def test_key_slices_fill_one_wave():
    """How many slices a decode step cuts its keys into: enough to fill one wave of CTAs, at
    least 512 keys each, one for prompts."""
    from types import SimpleNamespace

    from thintensor_b200.parts.attention import kv_splits

    def step(sequences, total, decode=True):
        return SimpleNamespace(decode=decode, max_total=total, sequences=sequences)

    assert kv_splits(step(8, 4096), 8 * 8, 512, 148) == 2           # 64 CTAs -> 128
    assert kv_splits(step(1, 2048), 8, 512, 148) == 4               # limited by 512 keys a slice
    assert kv_splits(step(1, 32768), 8, 512, 148) == 18             # 144 CTAs
    assert kv_splits(step(64, 2048), 64 * 8, 512, 148) == 1         # already several waves
    assert kv_splits(step(8, 4096, decode=False), 64, 512, 148) == 1
    assert kv_splits(step(1, 100), 8, 512, 148) == 1


def test_product_policies_need_no_device():
    """How a projection is run is decided on the host from its sizes alone: k-slices for few output
    tiles, none for CTA pairs, and the product added into the residual stream by the kernel wherever k is in
    one slice and tiled copies can do the adding (else only where every CTA has two tiles to hide the read under).  The number of multiprocessors is the device's at run
    time; here it is given (a B200 has 148)."""
    from thintensor_b200.kernels import api

    assert api.gemm_tcgen05_splits(8, 2048, 2048, sms=148) == 8 and api.gemm_tcgen05_splits(8, 128256, 2048, sms=148) == 1
    assert api.gemm_tcgen05_splits(512, 2048, 2048, sms=148) == 4 and api.gemm_tcgen05_splits(256, 2048, 2048, sms=148) == 4 and api.gemm_tcgen05_splits(2048, 2048, 8192, sms=148) == 1
    for tokens in (1, 8, 64, 128, 512, 1024):
        assert not api.gemm_tcgen05_accumulate_pays(tokens, 2048, 2048, sms=148), tokens       # 1B output projection: few tokens, or k in slices
    for tokens in (1536, 2048, 4096, 4736, 8192):                                              # one k-slice, rows that tiled copies can add to
        assert api.gemm_tcgen05_accumulate_pays(tokens, 2048, 2048, sms=148) and api.gemm_tcgen05_accumulate_pays(tokens, 2048, 8192, sms=148), tokens
    assert api.gemm_tcgen05_accumulate_pays(4096, 4096, 14336, sms=148) and api.gemm_tcgen05_accumulate_pays(2048, 4096, 14336, sms=148)
    # rows of 2,050 floats are added from registers after a read: only where a CTA pair has two tiles to hide it under
    assert not api.gemm_tcgen05_accumulate_pays(2048, 2050, 2048, sms=148) and api.gemm_tcgen05_accumulate_pays(4736, 2050, 2048, sms=148)
    assert api.gemm_tcgen05_accumulates(2048, 2050, 2048, sms=148) and not api.gemm_tcgen05_accumulates(512, 2048, 2048, sms=148)   # can, but does not pay; cannot (sliced)
    # whatever pays can be done
    for tokens in range(129, 9000, 371):
        for features, k in ((2048, 2048), (3072, 8192), (200, 64), (4096, 14336)):
            if api.gemm_tcgen05_accumulate_pays(tokens, features, k, sms=148):
                assert api.gemm_tcgen05_accumulates(tokens, features, k, sms=148) and api.gemm_tcgen05_splits(tokens, features, k, sms=148) == 1


def test_k_runs_of_cta_pairs_share_a_tile_among_at_most_three():
    """The CTA pairs' plain product may deal the tiles' k-blocks out as contiguous runs (units = tiles * k-blocks,
    pair p takes units [units * p // pairs, units * (p + 1) // pairs)).  The pair that holds a tile's first k-blocks adds
    at most two other pairs' shares, which the launcher guarantees by dealing only where tiles * 2 > pairs + 1
    (gemm_tcgen05.cu, deals_k_out and KRun): the arithmetic of that guarantee, for every size it admits."""
    for pairs in (2, 3, 66, 74):
        for k_blocks in (16, 17, 32, 48, 128, 224):
            for tiles in range(1, 4 * pairs + 3):
                if tiles * 2 <= pairs + 1:
                    continue
                units = tiles * k_blocks
                begins = [units * p // pairs for p in range(pairs + 1)]
                assert begins[0] == 0 and begins[-1] == units
                for tile in range(tiles):
                    lo, hi = tile * k_blocks, (tile + 1) * k_blocks
                    holders = [p for p in range(pairs) if begins[p] < hi and begins[p + 1] > lo]
                    assert 1 <= len(holders) <= 3, (pairs, k_blocks, tiles, tile, holders)
                    # only a pair's first item starts inside a tile: every holder but the first begins inside this tile
                    assert all(lo < begins[p] < hi for p in holders[1:])

"""The generation loop: requests in, token lists out.

``run_generation`` holds every decision of the loop and touches no device: which
requests form the next batch, when a sequence ends (a stop token, which is kept in the
output, or its token limit), that a sequence that ended leaves the batch and gives its
slot back at once, and that batches follow one another until no request is left.  It
drives a *backend* with four calls; :class:`EngineBackend` is the one that runs on the
GPU, tests use a scripted one.

The reference's loop serves one sequence: prompt tokens one at a time, then
``next_token -> EOS? -> forward_token`` with the EOS token kept in the output
(thinruntime/cli.py:2799-2858); its benchmark loop keeps sampled ids on the device and
never synchronises (scripts/thin_runtime.py:981-1011), which is what ``decode_run`` does
when there are no stop tokens.
"""
from __future__ import annotations

import time
import weakref
from dataclasses import dataclass, field
from typing import Protocol, Sequence

import torch

from ..kernels import api
from ..sampling.sampler import SamplingParams, sample
from .context import StepContext
from .engine import Engine, Entry


class GenerationError(ValueError):
    pass


MAX_DECODE_STATES = 16      # decode shapes whose captured steps an engine keeps


def table_width(blocks: int) -> int:
    """The width of a decode state's block tables for sequences of up to ``blocks`` blocks: the
    next power of two up to 16, then the next multiple of 16, so that batches whose lengths differ
    a little share a shape (and its captured step); entries beyond a sequence's blocks stay -1."""
    blocks = max(1, blocks)
    if blocks <= 16:
        return 1 << (blocks - 1).bit_length()
    return -(-blocks // 16) * 16


class Backend(Protocol):
    def fits(self, totals: Sequence[int]) -> bool:
        """Whether sequences that grow to these lengths can be live together."""

    def start_batch(self, requests: Sequence[int], prompts: Sequence[Sequence[int]], totals: Sequence[int]) -> list[int]:
        """Open a sequence for each prompt, run all prompts in one step and return the
        first new token of each.  ``requests`` are the requests' indices (they select
        the random numbers), ``totals`` the lengths the sequences may reach."""

    def decode_step(self, live: Sequence[int]) -> list[int]:
        """One more token for each of the batch's sequences named in ``live`` (positions
        in the batch), each fed the token it produced last."""

    def decode_run(self, live: Sequence[int], steps: int) -> list[list[int]]:
        """``steps`` decode steps without looking at the tokens in between; returns
        ``steps`` lists like ``decode_step``'s."""

    def finish(self, position: int) -> None:
        """The sequence at ``position`` of the batch has ended: free what it holds."""

    def abandon(self) -> None:
        """A call of the current batch raised: free what its unfinished sequences still hold,
        so that the error leaves the cache as it was before the batch."""


@dataclass
class GenerationStats:
    batches: int = 0
    prefill_steps: int = 0
    decode_steps: int = 0
    prompt_tokens: int = 0
    new_tokens: int = 0
    batch_sizes: list[int] = field(default_factory=list)
    prefill_seconds: float = 0.0            # host clock; every phase ends with tokens read on the host
    decode_seconds: float = 0.0
    decoded_tokens: int = 0                 # tokens produced by decode steps (the first of each request excluded)


def plan_batch(pending: list[int], totals: list[int], batch_size: int, backend: Backend) -> list[int]:
    """The requests (by index) of the next batch: the first ``batch_size`` pending ones,
    fewer if the cache cannot hold them together."""
    chosen: list[int] = []
    for index in pending:
        if len(chosen) == batch_size:
            break
        if not backend.fits([totals[i] for i in chosen] + [totals[index]]):
            break
        chosen.append(index)
    if not chosen:
        raise GenerationError(
            f"request {pending[0]} needs room for {totals[pending[0]]} tokens, more than the cache can hold even alone"
        )
    return chosen


def run_generation(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens: int, stop_ids: Sequence[int] = (),
                   batch_size: int = 8, context: int | None = None, stats: GenerationStats | None = None) -> list[list[int]]:
    """Generate up to ``max_new_tokens`` tokens for every prompt; returns the new tokens
    of each request, in request order."""
    if max_new_tokens <= 0:
        raise GenerationError(f"max_new_tokens must be positive, got {max_new_tokens}")
    if batch_size <= 0:
        raise GenerationError(f"batch_size must be positive, got {batch_size}")
    for index, prompt in enumerate(prompts):
        if len(prompt) == 0:
            raise GenerationError(f"prompt {index} is empty")
        if context is not None and len(prompt) + max_new_tokens > context:
            # the reference refuses the same way before running (thinruntime/cli.py:2788-2793)
            raise GenerationError(
                f"prompt {index} has {len(prompt)} tokens; with {max_new_tokens} new tokens it exceeds the context of {context}"
            )
    stats = stats if stats is not None else GenerationStats()
    stop = frozenset(int(s) for s in stop_ids)
    totals = [len(p) + max_new_tokens for p in prompts]
    results: list[list[int]] = [[] for _ in prompts]
    pending = list(range(len(prompts)))

    while pending:
        batch = plan_batch(pending, totals, batch_size, backend)
        pending = pending[len(batch):]
        try:
            _run_batch(backend, batch, prompts, totals, max_new_tokens, stop, results, stats)
        except BaseException:
            try:
                backend.abandon()
            except Exception:           # the first error is the one to report
                pass
            raise
    stats.new_tokens = sum(len(r) for r in results)
    return results


def _run_batch(backend: Backend, batch: list[int], prompts, totals: list[int], max_new_tokens: int, stop: frozenset,
               results: list[list[int]], stats: GenerationStats) -> None:
    """One batch from its prompts to the end of its last sequence."""
    stats.batches += 1
    stats.batch_sizes.append(len(batch))
    stats.prefill_steps += 1
    stats.prompt_tokens += sum(len(prompts[i]) for i in batch)
    clock = time.perf_counter()
    first = backend.start_batch(batch, [prompts[i] for i in batch], [totals[i] for i in batch])
    stats.prefill_seconds += time.perf_counter() - clock
    clock = time.perf_counter()
    live: list[int] = []                      # positions in the batch still running
    for position, (index, token) in enumerate(zip(batch, first)):
        results[index].append(int(token))
        if int(token) in stop or max_new_tokens == 1:
            backend.finish(position)
        else:
            live.append(position)
    produced = 1
    while live:
        if not stop:
            # nothing can end early: run to the limit without reading tokens back
            steps = max_new_tokens - produced
            for tokens in backend.decode_run(live, steps):
                for position, token in zip(live, tokens):
                    results[batch[position]].append(int(token))
            stats.decode_steps += steps
            stats.decoded_tokens += steps * len(live)
            for position in live:
                backend.finish(position)
            live = []
            break
        tokens = backend.decode_step(live)
        stats.decode_steps += 1
        stats.decoded_tokens += len(live)
        produced += 1
        still: list[int] = []
        for position, token in zip(live, tokens):
            results[batch[position]].append(int(token))
            if int(token) in stop or produced == max_new_tokens:
                backend.finish(position)
            else:
                still.append(position)
        live = still
    stats.decode_seconds += time.perf_counter() - clock


# --------------------------------------------------------------------------------------
# the backend that runs on the GPU
# --------------------------------------------------------------------------------------


class _DecodeState:
    """Device-resident description of a decode batch, so that a step needs nothing from
    the host: tokens (each step's samples are written where the next step reads them),
    lengths (advanced by a kernel), block tables, request ids and step counters.

    A state is made for a shape (number of sequences, width of the block tables) and filled
    for a batch; the graphs it captured serve every later batch of that shape, so only the
    first batch of a shape pays for the capture."""

    def __init__(self, engine: Engine, sequences: int, width: int):
        cache = engine.cache
        # The engine keeps its states, so a state must not keep the engine alive: a cycle would leave
        # the graphs to the garbage collector, and a graph destroyed while another is being captured
        # invalidates that capture.
        self._engine = weakref.ref(engine)
        self.sequences = b = sequences
        self.width = width
        self.max_total = width * cache.block_tokens          # bound of any length the tables can describe
        self.slots: list[int] = []
        groups = len(cache.kv_groups)
        self.groups = groups
        self.meta = torch.zeros(b + (b + 1) + b + b + groups * b * width + 3 * b, dtype=torch.int32, device=engine.device)
        p = 0

        def cut(n):
            nonlocal p
            view = self.meta[p : p + n]
            p += n
            return view

        self.tokens, self.cu, self.lengths, self.d_slots = cut(b), cut(b + 1), cut(b), cut(b)
        self.tables = [cut(b * self.width).view(b, self.width) for _ in range(groups)]
        self.rows, self.requests, self.steps = cut(b), cut(b), cut(b)
        self.graphs: dict[bool, tuple[torch.cuda.CUDAGraph, int]] = {}   # by whether the step copies tokens from and to the host
        pinned = torch.zeros(2 * b + 1, dtype=torch.int32, pin_memory=True)
        self.host_in, self.host_out = pinned[:b], pinned[b:]  # tokens fed by the host; tokens sampled, then the status word
        self.feed = self.host_in.numpy()                      # the same memory, written without a tensor in between
        self.fetched = self.host_out.numpy()
        self.warm = False
        self.logits: torch.Tensor | None = None  # the last step's logits
        self.launches_per_step = 0              # kernels of this library in one decode step

    @property
    def engine(self) -> Engine:
        engine = self._engine()
        if engine is None:
            raise GenerationError("the engine of this decode state is gone")
        return engine

    def fill(self, slots: list[int], requests: list[int], last_tokens: list[int], steps_done: list[int], totals: list[int]) -> None:
        """Describe a batch: its slots, the token each sequence is fed next, its length, the
        blocks it may grow into (reserved here, so the tables stay as they are for the run)."""
        cache = self.engine.cache
        b = self.sequences
        if len(slots) != b or max(-(-t // cache.block_tokens) for t in totals) > self.width:
            raise GenerationError("the batch does not have the shape this decode state was made for")
        self.slots = list(slots)
        for slot, total in zip(slots, totals):
            cache.reserve(slot, total)
        flat: list[int] = []
        flat.extend(last_tokens)                # tokens
        flat.extend(range(b + 1))               # cu
        flat.extend(cache.length(s) for s in slots)
        flat.extend(slots)
        for g in range(self.groups):
            for row in cache.table_rows(g, slots, self.width):
                flat.extend(row)
        flat.extend(range(b))                   # rows: every token's logits
        flat.extend(requests)
        flat.extend(steps_done)
        self.meta.copy_(torch.tensor(flat, dtype=torch.int32))

    def context(self) -> StepContext:
        e = self.engine
        return StepContext(
            n_tokens=self.sequences, sequences=self.sequences, decode=True, max_new=1, max_total=self.max_total,
            tokens=self.tokens, cu=self.cu, len_before=self.lengths, slots=self.d_slots, tables=self.tables,
            act_dtype=e.model.dtype, workspace=e.workspace, status=e.status, host_slots=self.slots,
            host_new=[1] * self.sequences, host_before=[],
        )

    def body(self, params: SamplingParams) -> None:
        """One decode step, entirely on the device."""
        e = self.engine
        logits = e.model.forward(self.context(), e.cache, self.rows)
        self.logits = logits                    # float32 [sequences, vocab]; a replayed step writes to the same place
        sample(logits, params, self.requests, self.steps, self.tokens)
        api.advance_lengths(self.lengths, self.cu, self.sequences, self.steps)

    def body_with_host(self, params: SamplingParams) -> None:
        """The step with the host as the authority on tokens: ``host_in`` goes up before it,
        the samples come down into ``host_out`` after it together with the device status word, both
        by small kernels that address the pinned host memory (a copy node in a graph costs several
        times as much)."""
        api.copy_int32(self.tokens, self.host_in)
        self.body(params)
        api.copy_int32(self.host_out, self.tokens, self.engine.status)

    def step(self, params: SamplingParams, use_graph: bool, host_io: bool = False) -> None:
        e = self.engine
        body = self.body_with_host if host_io else self.body
        if not use_graph or not self.warm:
            before = api.launch_count()
            body(params)                        # the first run also allocates scratch and compiles
            self.launches_per_step = api.launch_count() - before
            self.warm = True
        else:
            graph, generation = self.graphs.get(host_io, (None, -1))
            if graph is None or generation != e.workspace.generation:     # a graph holds the addresses of scratch memory
                generation = e.workspace.generation
                graph = torch.cuda.CUDAGraph()
                # capture replays nothing; the captured step runs at the first replay
                with torch.cuda.graph(graph):
                    body(params)
                if e.workspace.generation != generation:
                    raise RuntimeError("scratch memory moved while a decode step was being captured")
                self.graphs[host_io] = (graph, generation)
            graph.replay()
        for slot in self.slots:
            e.cache.advance(slot, 1)


class EngineBackend:
    """Runs the loop's calls on an :class:`Engine`."""

    def __init__(self, engine: Engine, params: SamplingParams, use_graph: bool = True):
        self.engine = engine
        self.params = params
        self.use_graph = use_graph
        self._slots: list[int | None] = []
        self._requests: list[int] = []
        self._totals: list[int] = []
        self._last: list[int] = []
        self._steps: list[int] = []
        self._state: _DecodeState | None = None
        self._state_live: tuple[int, ...] = ()

    def fits(self, totals: Sequence[int]) -> bool:
        cache = self.engine.cache
        blocks = sum(-(-t // cache.block_tokens) for t in totals)
        return blocks <= cache.free_blocks and len(totals) <= cache.slots.free_count

    def start_batch(self, requests, prompts, totals) -> list[int]:
        e = self.engine
        self._slots = []
        for _ in prompts:                       # one by one: if the cache runs out of slots, abandon() finds the earlier ones
            self._slots.append(e.open())
        self._requests, self._totals = list(requests), list(totals)
        self._steps = [1] * len(prompts)
        self._state = None
        for slot, total in zip(self._slots, totals):
            e.cache.reserve(slot, total)
        logits = e.step([Entry(slot, list(prompt), [len(prompt) - 1]) for slot, prompt in zip(self._slots, prompts)])
        out = torch.empty(len(prompts), dtype=torch.int32, device=e.device)
        request = torch.tensor(self._requests, dtype=torch.int32, device=e.device)
        step = torch.zeros(len(prompts), dtype=torch.int32, device=e.device)
        sample(logits, self.params, request, step, out)
        self._last = out.tolist()
        e.check_status()
        return list(self._last)

    def _state_for(self, live: Sequence[int]) -> _DecodeState:
        key = tuple(live)
        if self._state is None or self._state_live != key:
            e = self.engine
            totals = [self._totals[p] for p in live]
            width = table_width(max(-(-t // e.cache.block_tokens) for t in totals))
            # states and their graphs are kept with the engine, by everything a captured step holds as a constant
            shape = (len(live), width, self.params)
            state = e.decode_states.pop(shape, None)
            if state is None:
                state = _DecodeState(e, len(live), width)
                while len(e.decode_states) >= MAX_DECODE_STATES:
                    e.decode_states.pop(next(iter(e.decode_states)))       # the one used longest ago
            e.decode_states[shape] = state                                  # most recently used last
            state.fill([self._slots[p] for p in live], [self._requests[p] for p in live], [self._last[p] for p in live],
                       [self._steps[p] for p in live], totals)
            self._state, self._state_live = state, key
        return self._state

    def decode_step(self, live) -> list[int]:
        """The host is the authority on what each sequence is fed: the last tokens go up
        from pinned memory, the new ones come back, every step."""
        state = self._state_for(live)
        state.feed[:] = [self._last[p] for p in live]
        state.step(self.params, self.use_graph, host_io=True)
        torch.cuda.current_stream(self.engine.device).synchronize()
        fetched = state.fetched.tolist()
        tokens, status = fetched[:-1], fetched[-1]
        if status:
            # a kernel of this step flagged a fault: the tokens are not to be trusted, and the sequence
            # that caused it is in this batch, not in a later one
            self.engine.check_status()
        for position, token in zip(live, tokens):
            self._last[position] = token
            self._steps[position] += 1
        return tokens

    def decode_run(self, live, steps: int) -> list[list[int]]:
        if steps <= 0:
            return []
        state = self._state_for(live)
        history = torch.empty((steps, len(live)), dtype=torch.int32, device=self.engine.device)
        for i in range(steps):
            state.step(self.params, self.use_graph)
            api.copy_int32(history[i], state.tokens)
        out = history.tolist()
        for position, token in zip(live, out[-1]):
            self._last[position] = token
            self._steps[position] += steps
        self.engine.check_status()
        return out

    def finish(self, position: int) -> None:
        slot = self._slots[position]
        if slot is None:
            raise GenerationError(f"the sequence at position {position} was finished twice")
        self.engine.close(slot)
        self._slots[position] = None
        self._state = None

    def abandon(self) -> None:
        for position, slot in enumerate(self._slots):
            if slot is not None:
                self.engine.close(slot)
                self._slots[position] = None
        self._state = None

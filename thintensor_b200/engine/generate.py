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
from dataclasses import dataclass, field
from typing import Protocol, Sequence

import torch

from ..kernels import api
from ..sampling.sampler import SamplingParams, sample
from .context import StepContext
from .engine import Engine, Entry


class GenerationError(ValueError):
    pass


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
    stats.new_tokens = sum(len(r) for r in results)
    return results


# --------------------------------------------------------------------------------------
# the backend that runs on the GPU
# --------------------------------------------------------------------------------------


class _DecodeState:
    """Device-resident description of a decode batch, so that a step needs nothing from
    the host: tokens (each step's samples are written where the next step reads them),
    lengths (advanced by a kernel), block tables, request ids and step counters."""

    def __init__(self, engine: Engine, slots: list[int], requests: list[int], last_tokens: list[int], steps_done: list[int],
                 totals: list[int]):
        cache = engine.cache
        self.engine = engine
        self.slots = list(slots)
        self.sequences = b = len(slots)
        self.width = max(1, max(-(-t // cache.block_tokens) for t in totals))
        groups = len(cache.kv_groups)
        for slot, total in zip(slots, totals):
            cache.reserve(slot, total)          # tables stay as they are for the whole run
        flat: list[int] = []
        flat.extend(last_tokens)                # tokens
        flat.extend(range(b + 1))               # cu
        flat.extend(cache.length(s) for s in slots)
        flat.extend(slots)
        for g in range(groups):
            for row in cache.table_rows(g, slots, self.width):
                flat.extend(row)
        flat.extend(range(b))                   # rows: every token's logits
        flat.extend(requests)
        flat.extend(steps_done)
        self.meta = torch.tensor(flat, dtype=torch.int32).to(engine.device)
        p = 0

        def cut(n):
            nonlocal p
            view = self.meta[p : p + n]
            p += n
            return view

        self.tokens, self.cu, self.lengths, self.d_slots = cut(b), cut(b + 1), cut(b), cut(b)
        self.tables = [cut(b * self.width).view(b, self.width) for _ in range(groups)]
        self.rows, self.requests, self.steps = cut(b), cut(b), cut(b)
        self.max_total = max(totals)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.warm = False
        self.launches_per_step = 0              # kernels of this library in one decode step

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
        sample(logits, params, self.requests, self.steps, self.tokens)
        api.advance_lengths(self.lengths, self.cu, self.sequences)
        self.steps.add_(1)

    def step(self, params: SamplingParams, use_graph: bool) -> None:
        e = self.engine
        if not use_graph or not self.warm:
            before = api.launch_count()
            self.body(params)                   # the first run also allocates scratch and compiles
            self.launches_per_step = api.launch_count() - before
            self.warm = True
        else:
            if self.graph is None:
                generation = e.workspace.generation
                graph = torch.cuda.CUDAGraph()
                # capture replays nothing; the captured step runs at the first replay
                with torch.cuda.graph(graph):
                    self.body(params)
                if e.workspace.generation != generation:
                    raise RuntimeError("scratch memory moved while a decode step was being captured")
                self.graph = graph
            self.graph.replay()
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
        self._pinned: torch.Tensor | None = None

    def fits(self, totals: Sequence[int]) -> bool:
        cache = self.engine.cache
        blocks = sum(-(-t // cache.block_tokens) for t in totals)
        return blocks <= cache.free_blocks and len(totals) <= cache.slots.free_count

    def start_batch(self, requests, prompts, totals) -> list[int]:
        e = self.engine
        self._slots = [e.open() for _ in prompts]
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
            self._state = _DecodeState(
                self.engine, [self._slots[p] for p in live], [self._requests[p] for p in live], [self._last[p] for p in live],
                [self._steps[p] for p in live], [self._totals[p] for p in live],
            )
            self._state_live = key
        return self._state

    def decode_step(self, live) -> list[int]:
        """The host is the authority on what each sequence is fed: the last tokens go up
        from pinned memory, the new ones come back, every step."""
        state = self._state_for(live)
        if self._pinned is None or self._pinned.numel() < len(live):
            self._pinned = torch.empty(max(64, len(live)), dtype=torch.int32, pin_memory=True)
        feed = self._pinned[: len(live)]
        feed.copy_(torch.tensor([self._last[p] for p in live], dtype=torch.int32))
        state.tokens.copy_(feed, non_blocking=True)
        state.step(self.params, self.use_graph)
        tokens = state.tokens.tolist()
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
            history[i].copy_(state.tokens)
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

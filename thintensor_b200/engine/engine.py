"""The step function: a batch of sequences, the tokens each brings, logits at the wanted
places.

``Engine.step`` runs only the tokens it is given, as one packed batch, against the
cache that earlier steps left, and advances the sequences.  Sequences of a step may
bring different numbers of tokens (their prompts, or one token each); nothing is padded.
A step with more packed tokens than ``max_step_tokens`` is cut along the token axis
into pieces that run one after another: later pieces find the earlier pieces' keys in
the cache, so the result does not depend on the cut.

The reference's only entry is one token of one sequence per call,
``forward_token(token_id, token_index) -> hidden`` followed by ``logits(hidden)``
(thinruntime/gpu_runtime.py:7599-7633, 11006-11087), with the prompt fed through it in a
Python loop (thinruntime/cli.py:2802-2807).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..cache.cache import SequenceCache
from ..kernels import api
from .context import StepContext, Workspace
from .model import DecoderModel


@dataclass
class Entry:
    """One sequence's share of a step: its slot, its next tokens, and the places among
    these tokens whose logits are wanted."""

    slot: int
    tokens: list[int]           # or a one-dimensional integer numpy array
    want: list[int]


class StepError(ValueError):
    pass


class _Staging:
    """Pinned host buffers for a step's integers, reused in rotation; a buffer is not
    rewritten before the copy that last read it has finished."""

    def __init__(self, count: int = 4):
        self._buffers: list[torch.Tensor | None] = [None] * count
        self._events: list[torch.cuda.Event | None] = [None] * count
        self._next = 0

    def take(self, n_ints: int) -> tuple[torch.Tensor, int]:
        index = self._next
        self._next = (self._next + 1) % len(self._buffers)
        if self._events[index] is not None:
            self._events[index].synchronize()
        buffer = self._buffers[index]
        if buffer is None or buffer.numel() < n_ints:
            buffer = torch.empty(max(n_ints, 1024), dtype=torch.int32, pin_memory=True)
            self._buffers[index] = buffer
        return buffer, index

    def sent(self, index: int) -> None:
        event = self._events[index] or torch.cuda.Event()
        event.record()
        self._events[index] = event


MAX_STEP_GRAPHS = 32         # shapes of steps whose captured launches an engine keeps
MAX_GRAPH_ROWS = 64          # a step that wants more logits rows than this is not replayed (its rows are copied once more)


@dataclass
class _StepGraph:
    """A step shape's kernels, captured once: replaying them costs the host one call instead of one
    per kernel.  ``logits`` is where the captured step leaves its wanted rows."""

    graph: torch.cuda.CUDAGraph | None      # None: the shape has run once, eagerly; its next step is captured
    generation: int = -1                    # of the scratch memory whose addresses the graph holds
    logits: torch.Tensor | None = None


class Engine:
    def __init__(self, model: DecoderModel, cache: SequenceCache, max_step_tokens: int = 8192, step_graphs: bool = True):
        if model.device is None or model.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        if not model.bound:
            raise RuntimeError("the model has no weights yet")
        self.model = model
        self.cache = cache
        self.device = model.device
        self.max_step_tokens = int(max_step_tokens)
        self.workspace = Workspace(self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._staging = _Staging()
        self.vocab_size = model.spec.vocab_size
        self.launch_count = 0
        self.decode_states: dict = {}        # the generation loop's captured decode steps, by shape
        # Steps through `step` of a shape that has run before are replayed from a CUDA graph: everything that
        # differs between two steps of one shape (tokens, lengths, slots, tables, wanted rows) is device data.
        self.step_graphs: dict[tuple, _StepGraph] = {}
        self.use_step_graphs = bool(step_graphs) and model.device_driven
        self.graph_replays = 0

    # ------------------------------------------------------------- sequences
    def open(self) -> int:
        """Start a sequence: a free slot with no tokens."""
        return self.cache.alloc_slot()

    def close(self, slot: int) -> None:
        """End a sequence: its slot and blocks go back to the cache."""
        self.cache.free_slot(slot)

    # ------------------------------------------------------------------ step
    def validate(self, entries: list[Entry]) -> list[np.ndarray]:
        """Check a step on the host and return every entry's tokens as an int32 array (made once
        here, so that the range check and the copy to the device need no second pass over the list)."""
        arrays: list[np.ndarray] = []
        if not entries:
            raise StepError("a step needs at least one sequence")
        seen: set[int] = set()
        for entry in entries:
            if entry.slot in seen:
                raise StepError(f"slot {entry.slot} appears twice in one step")
            seen.add(entry.slot)
            self.cache.length(entry.slot)  # raises if the slot is not live
            if len(entry.tokens) == 0:
                raise StepError(f"slot {entry.slot} brings no tokens")
            try:
                if isinstance(entry.tokens, np.ndarray) and entry.tokens.dtype.kind in "iu" and entry.tokens.ndim == 1:
                    tokens = entry.tokens.astype(np.int64, copy=False)     # an integer array is taken as it is (a list costs 30 ns a token)
                else:
                    tokens = np.fromiter(entry.tokens, dtype=np.int64, count=len(entry.tokens))
            except (OverflowError, TypeError, ValueError) as exc:
                raise StepError(f"slot {entry.slot}: token ids must be integers ({exc})") from None
            if tokens.min() < 0 or tokens.max() >= self.vocab_size:
                token = next(int(t) for t in entry.tokens if not 0 <= t < self.vocab_size)
                raise StepError(f"token id {token} is outside the vocabulary of {self.vocab_size}")
            arrays.append(tokens.astype(np.int32))
            if entry.want and (min(entry.want) < 0 or max(entry.want) >= len(entry.tokens)):
                place = next(p for p in entry.want if not 0 <= p < len(entry.tokens))
                raise StepError(f"wanted place {place} is outside the {len(entry.tokens)} tokens slot {entry.slot} brings")
        return arrays

    def step(self, entries: list[Entry]) -> torch.Tensor:
        """Run the entries' tokens and return float32 logits ``[wanted, vocab]`` on the
        device, ordered by entry and then by ``want``."""
        arrays = self.validate(entries)
        for entry in entries:
            self.cache.reserve(entry.slot, self.cache.length(entry.slot) + len(entry.tokens))
        total_wanted = sum(len(e.want) for e in entries)
        out = torch.empty((total_wanted, self.vocab_size), dtype=torch.float32, device=self.device)
        out_base = []
        running = 0
        for entry in entries:
            out_base.append(running)
            running += len(entry.want)

        pieces = self._pieces(entries)
        for piece in pieces:
            replayable = self.use_step_graphs and len(pieces) == 1 and total_wanted <= MAX_GRAPH_ROWS
            ctx, rows, targets = self._prepare(entries, arrays, piece, out_base, replayable)
            if replayable:
                logits = self._forward_replayed(ctx, rows)
                if logits is not None:
                    out.copy_(logits)               # one piece: its wanted rows are the result's rows, in order
            elif rows is not None:
                if len(pieces) == 1:
                    ctx.logits_out = out            # one piece: its wanted rows are the result's rows, in order
                logits = self.model.forward(ctx, self.cache, rows)
                if logits.data_ptr() != out.data_ptr() or logits.shape != out.shape:
                    out.index_copy_(0, targets.to(torch.int64), logits)
            else:
                self._forward_without_logits(ctx)
            for index, start, count in piece:
                self.cache.advance(entries[index].slot, count)
        return out

    def _forward_replayed(self, ctx: StepContext, rows: torch.Tensor | None) -> torch.Tensor | None:
        """Run a one-piece step whose shape is its key: eagerly the first time, captured into a CUDA graph
        the second time, replayed from then on (and captured again if scratch memory has moved since).
        The step's integers are already in their place on the device; the wanted rows come back in a
        buffer of the engine's."""
        n_rows = 0 if rows is None else rows.numel()
        key = (ctx.n_tokens, ctx.sequences, tuple(t.shape[1] for t in ctx.tables), n_rows, ctx.decode)
        if n_rows:
            ctx.logits_out = self.workspace.get("step.logits", (n_rows, self.vocab_size), torch.float32)
        entry = self.step_graphs.get(key)
        if entry is None:
            while len(self.step_graphs) >= MAX_STEP_GRAPHS:
                self.step_graphs.pop(next(iter(self.step_graphs)))          # the one used longest ago
            self.step_graphs[key] = _StepGraph(None)
            return self.model.forward(ctx, self.cache, rows)
        self.step_graphs[key] = self.step_graphs.pop(key)                   # most recently used last
        if entry.graph is None or entry.generation != self.workspace.generation:
            entry.generation = self.workspace.generation
            entry.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(entry.graph):                             # captures; the step runs at the replay below
                entry.logits = self.model.forward(ctx, self.cache, rows)
            if self.workspace.generation != entry.generation:
                self.step_graphs.pop(key)
                raise RuntimeError("scratch memory moved while a step was being captured")
        entry.graph.replay()
        self.graph_replays += 1
        return entry.logits

    def check_status(self) -> None:
        """Read the device status word (synchronises) and raise if a kernel flagged a
        fault during the steps since the last check."""
        word = int(self.status.item())
        if word:
            self.status.zero_()
            self.workspace.zero_again()         # tickets and flags that a kernel which gave up may have left set
            names = []
            if word & api.STATUS_BAD_TOKEN:
                names.append("a token id outside the vocabulary reached the embedding")
            if word & api.STATUS_BAD_BLOCK:
                names.append("a block table entry outside the pool was met")
            if word & api.STATUS_WAIT_EXPIRED:
                names.append("a bounded wait inside a kernel ran out")
            if word & api.STATUS_BAD_SHAPE:
                names.append("a kernel was given a size it cannot take")
            raise RuntimeError("device status " + hex(word) + ": " + "; ".join(names))

    # -------------------------------------------------------------- internals
    def _pieces(self, entries: list[Entry]) -> list[list[tuple[int, int, int]]]:
        """Cut the step along the packed token axis: each piece is a list of
        (entry index, first token, count)."""
        pieces: list[list[tuple[int, int, int]]] = [[]]
        room = self.max_step_tokens
        for index, entry in enumerate(entries):
            start = 0
            while start < len(entry.tokens):
                if room == 0:
                    pieces.append([])
                    room = self.max_step_tokens
                count = min(room, len(entry.tokens) - start)
                pieces[-1].append((index, start, count))
                start += count
                room -= count
        return pieces

    def _prepare(self, entries, arrays, piece, out_base, replayable: bool = False):
        slots = [entries[i].slot for i, _, _ in piece]
        before = [self.cache.length(s) for s in slots]
        new = [count for _, _, count in piece]
        n_tokens = sum(new)
        sequences = len(piece)
        rows: list[int] = []
        targets: list[int] = []
        offset = 0
        for (index, start, count) in piece:
            entry = entries[index]
            for k, place in enumerate(entry.want):
                if start <= place < start + count:
                    rows.append(offset + place - start)
                    targets.append(out_base[index] + k)
            offset += count
        cu = [0]
        for count in new:
            cu.append(cu[-1] + count)
        width = max(1, self.cache.max_blocks(slots))
        groups = len(self.cache.kv_groups)

        n_ints = n_tokens + (sequences + 1) + 2 * sequences + groups * sequences * width + 2 * len(rows)
        host, staging_index = self._staging.take(n_ints)
        device = self.workspace.get("step.meta", (n_ints,), torch.int32)
        staged = host.numpy()
        at = 0
        for (index, start, count) in piece:                      # the tokens: array to pinned memory, no Python loop
            staged[at : at + count] = arrays[index][start : start + count]
            at += count
        flat: list[int] = []
        flat.extend(cu)
        flat.extend(before)
        flat.extend(slots)
        for g in range(groups):
            for row in self.cache.table_rows(g, slots, width):
                flat.extend(row)
        flat.extend(rows)
        flat.extend(targets)
        staged[n_tokens:n_ints] = flat
        device.copy_(host[:n_ints], non_blocking=True)
        self._staging.sent(staging_index)

        p = 0
        def cut(n):
            nonlocal p
            view = device[p : p + n]
            p += n
            return view
        d_tokens, d_cu, d_before, d_slots = cut(n_tokens), cut(sequences + 1), cut(sequences), cut(sequences)
        d_tables = [cut(sequences * width).view(sequences, width) for _ in range(groups)]
        d_rows = cut(len(rows)) if rows else None
        d_targets = cut(len(rows)) if rows else None
        ctx = StepContext(
            n_tokens=n_tokens, sequences=sequences, decode=all(c == 1 for c in new), max_new=max(new),
            # a step that may be replayed must not bake this step's lengths into its launches: the bound is what the tables can describe
            max_total=width * self.cache.block_tokens if replayable else max(b + c for b, c in zip(before, new)), tokens=d_tokens, cu=d_cu, len_before=d_before, slots=d_slots,
            tables=d_tables, act_dtype=self.model.dtype, workspace=self.workspace, status=self.status,
            host_slots=slots, host_new=new, host_before=before,
        )
        return ctx, d_rows, d_targets

    def _forward_without_logits(self, ctx: StepContext) -> None:
        """A piece none of whose logits are wanted still has to fill the cache; it runs
        without the final norm and the head."""
        self.model.forward(ctx, self.cache, None)

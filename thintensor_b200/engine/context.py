"""What a part sees of a step: the packed tokens, where each sequence's tokens start,
how long each sequence was before the step, the block tables, and scratch memory.

A step runs ``n_tokens`` packed tokens of ``sequences`` sequences.  Token ``t`` belongs
to the sequence ``b`` with ``cu[b] <= t < cu[b + 1]`` and stands at position
``len_before[b] + t - cu[b]``.  All of these live on the device, so a decode step
captured in a CUDA graph can be replayed while a kernel advances the lengths.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


class Workspace:
    """Named scratch buffers that persist between steps.  A buffer grows when a step
    asks for more than it holds and otherwise keeps its address, so steps of a shape
    that has run before allocate nothing (a requirement for graph replay).  A buffer that
    has to grow at least doubles, so a run of slightly longer and longer steps moves it
    (and makes every captured decode step be captured again) only a few times."""

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: dict[str, torch.Tensor] = {}
        self._views: dict[tuple, torch.Tensor] = {}   # (name, shape, dtype) -> the view handed out last time
        self.generation = 0  # bumped whenever a buffer moves
        self._zeroed: set[str] = set()                # names handed out by get_zeroed

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (name, shape, dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        count = 1
        for s in shape:
            count *= int(s)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        buffer = self._buffers.get(name)
        if buffer is None or buffer.numel() < nbytes:
            grow = max(nbytes, 2 * buffer.numel() if buffer is not None else 0, 256)
            grow = -(-grow // 256) * 256
            buffer = None                                                    # the old one goes before the new one comes
            self._buffers.pop(name, None)
            buffer = torch.empty(grow, dtype=torch.uint8, device=self.device)
            self._buffers[name] = buffer
            self.generation += 1
            self._views = {k: v for k, v in self._views.items() if k[0] != name}   # views of the old buffer
        view = buffer[:nbytes].view(dtype).view(*shape)
        if len(self._views) < 4096:
            self._views[key] = view
        return view

    def get_zeroed(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Like :meth:`get`, for a buffer that is zero when it is first handed out (and again whenever it has had
        to move); afterwards its users leave it as they found it."""
        buffer = self._buffers.get(name)
        view = self.get(name, shape, dtype)
        if self._buffers.get(name) is not buffer:
            self._buffers[name].zero_()
        self._zeroed.add(name)
        return view

    def zero_again(self) -> None:
        """After a kernel gave up (a bounded wait that ran out, a size it refused) the users of these buffers may not
        have left them as they found them: tickets half drawn, flags set by a CTA whose partner had stopped waiting."""
        for name in self._zeroed:
            buffer = self._buffers.get(name)
            if buffer is not None:
                buffer.zero_()

    def bytes(self) -> int:
        return sum(b.numel() for b in self._buffers.values())


@dataclass
class StepContext:
    n_tokens: int                       # packed tokens in this step
    sequences: int                      # sequences in this step
    decode: bool                        # every sequence brings exactly one token
    max_new: int                        # most tokens any sequence brings
    max_total: int                      # upper bound of any sequence's length after the step
    tokens: torch.Tensor                # int32 [n_tokens]
    cu: torch.Tensor                    # int32 [sequences + 1]
    len_before: torch.Tensor            # int32 [sequences]
    slots: torch.Tensor                 # int32 [sequences], for per-sequence state
    tables: list[torch.Tensor]          # per KV group: int32 [sequences, width]
    act_dtype: torch.dtype              # dtype of activations and of the cache
    workspace: Workspace
    status: torch.Tensor                # uint32-as-int32 [1] device status word
    host_slots: list[int] = field(default_factory=list)
    host_new: list[int] = field(default_factory=list)       # tokens each sequence brings
    host_before: list[int] = field(default_factory=list)    # lengths before the step (unknown inside a replayed graph)
    logits_out: torch.Tensor | None = None                  # float32 [wanted rows, vocab] the head may write directly
    residual: torch.Tensor | None = None                    # float32 [n_tokens, hidden]: set by an arrangement whose parts may add into the stream themselves
    memo: dict = field(default_factory=dict)                # what a part computed for this step that its other layers can use again

    def scratch(self, name: str, shape: tuple[int, ...], dtype: torch.dtype | None = None) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype or self.act_dtype)

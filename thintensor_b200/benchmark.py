"""Timing prefill and decode steps on the device, with what a roofline needs.

The method is the reference's (scripts/thin_runtime.py:907-1011): warm-up steps, then a
timed loop bracketed by CUDA events with no host synchronisation inside and sampled
ids kept on the device.  A decode step reads every weight once (more than the L2
holds), so consecutive timed steps cannot serve each other from cache.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .engine.engine import Entry
from .engine.generate import EngineBackend, _DecodeState
from .kernels import api
from .sampling.sampler import SamplingParams

# Named shapes for benchmarks with random weights, each a whole config.json: the three Llama 3
# models the reference's reports measure and two tiny ones that differ in every size and option.
# They are data (config/shapes.json), read here and by bench.py.
SHAPES: dict[str, dict] = json.loads((Path(__file__).resolve().parent / "config" / "shapes.json").read_text(encoding="utf-8"))


def weight_bytes_per_step(model) -> int:
    """Bytes of weights a decode step reads: every matrix and vector once; of the
    embedding table only when it also serves as the head."""
    seen: set[int] = set()
    total = 0

    def add(t):
        nonlocal total
        if t is not None and t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()

    for arrangement in model.layers:
        for part in arrangement.parts.values():
            for value in vars(part).values():
                for linear in (value, getattr(value, "fused", None)):
                    if hasattr(linear, "weight") and hasattr(linear, "out_features"):
                        add(linear.weight)
                        add(linear.bias)
            if hasattr(part, "weight") and isinstance(part.weight, torch.Tensor):
                add(part.weight)
    add(model.head.part.linear.weight)
    add(model.final_norm.part.weight)
    return total


def kv_bytes_per_token(model) -> int:
    """Bytes of keys and values one cached token takes over all layers."""
    kv, _, source = model.cache_needs()
    width = torch.empty((), dtype=model.dtype).element_size()
    return sum(2 * need.kv_heads * need.head_dim * width for need, src in zip(kv, source) if need is not None)


def linear_flops_per_token(model) -> int:
    """Multiply-adds times two of all projections for one token (the head excluded)."""
    total = 0
    for run in model.spec.schedule:
        for part in model.layers[run.layer].parts.values():
            for value in vars(part).values():
                for linear in (value, getattr(value, "fused", None)):
                    if hasattr(linear, "out_features"):
                        total += 2 * linear.out_features * linear.in_features
    return total


def prefill_flops(model, tokens: int) -> float:
    """Projections for every token, causal attention (QK^T and PV over t(t+1)/2 pairs),
    and the head at one position."""
    flops = float(linear_flops_per_token(model)) * tokens
    kv, _, _ = model.cache_needs()
    for run, need in zip(model.spec.schedule, kv):
        if need is None:
            continue
        mixer = model.layers[run.layer].mixer()
        flops += 2.0 * 2.0 * (tokens * (tokens + 1) / 2) * need.head_dim * mixer.heads
    flops += 2.0 * model.spec.vocab_size * model.spec.hidden_size
    return flops


def measure_prefill(runtime, prompt: list[int], repeats: int = 3, warmup: int = 2) -> dict:
    """One sequence's whole prompt in one step, logits at its last position."""
    engine = runtime.new_engine(max_tokens=len(prompt) + 64, max_sequences=1, max_step_tokens=max(8192, len(prompt)))
    times = []
    for i in range(warmup + repeats):
        slot = engine.open()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([Entry(slot, prompt, [len(prompt) - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.close(slot)
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    engine.check_status()
    ms = sum(times) / len(times)
    return {"ms": ms, "tokens": len(prompt), "tokens_per_s": len(prompt) / (ms / 1e3), "flops": prefill_flops(runtime.model, len(prompt))}


def measure_decode(runtime, prompts: list[list[int]], context: int, warmup: int, steps: int, use_graph: bool = True) -> dict:
    """Prefill ``prompts`` together, then time ``steps`` greedy decode steps of the whole
    batch (after ``warmup`` untimed ones) with CUDA events."""
    batch = len(prompts)
    longest = max(len(p) for p in prompts)
    if longest + warmup + steps + 1 > context:
        raise ValueError(f"prompt {longest} + warmup {warmup} + steps {steps} does not fit the context {context}")
    per_sequence = -(-context // 64) * 64
    engine = runtime.new_engine(max_tokens=per_sequence * batch, max_sequences=batch)
    backend = EngineBackend(engine, SamplingParams(), use_graph)
    backend.start_batch(list(range(batch)), prompts, [context] * batch)
    live = list(range(batch))
    state: _DecodeState = backend._state_for(live)
    params = backend.params
    for _ in range(max(warmup, 2)):                 # the second step captures the graph
        state.step(params, use_graph)
    torch.cuda.synchronize()
    launches_before = api.launch_count()
    if use_graph and not state.graphs:
        state.step(params, use_graph)
    lengths_before = [engine.cache.length(s) for s in state.slots]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        state.step(params, use_graph)
    stop.record()
    torch.cuda.synchronize()
    engine.check_status()
    ms = start.elapsed_time(stop)
    mean_context = sum(lengths_before) / batch + (steps - 1) / 2.0
    bytes_per_step = weight_bytes_per_step(runtime.model) + kv_bytes_per_token(runtime.model) * mean_context * batch
    result = {
        "ms_per_step": ms / steps,
        "tokens_per_s": batch * steps / (ms / 1e3),
        "batch": batch,
        "mean_context": mean_context,
        "bytes_per_step": bytes_per_step,
        "launches_per_step": state.launches_per_step,
        "eager_launches": api.launch_count() - launches_before,
    }
    for position in live:
        backend.finish(position)
    return result

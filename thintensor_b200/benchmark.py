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


FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks(file: str | Path | None = None) -> dict:
    """The denominators of the roofline fractions: a measured copy bandwidth (GB/s) and a measured
    dense bfloat16 matrix-product rate (TFLOP/s) from ``file`` (JSON with ``hbm_gbs`` and
    ``bf16_tflops``; default ``MEASURED_PEAKS.json`` in the working directory) if it exists, else
    an earlier measurement on a B200 (6.65 TB/s, 1.59 PFLOP/s), marked ``fallback``."""
    path = Path(file) if file is not None else Path("MEASURED_PEAKS.json")
    if path.is_file():
        raw = json.loads(path.read_text(encoding="utf-8"))
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
    if file is not None:
        raise FileNotFoundError(f"no peaks file at {path}")
    return dict(FALLBACK_PEAKS)


def _tensor_bytes(t) -> int:
    return 0 if t is None else t.numel() * t.element_size()


def _step_parts(model):
    """Every part a step runs, once per run of the schedule, then the final norm and the head.
    The embedding is left out: a step gathers one row per token from it."""
    for run in model.spec.schedule:
        yield from model.layers[run.layer].parts.values()
    yield model.final_norm.part
    yield model.head.part


def weight_bytes_per_step(model) -> int:
    """Bytes of weights a decode step reads: every projection (``Part.projections``) and every
    vector (``Part.vectors``) of every run once.  A tied head is the embedding table, which is
    counted there, as the head."""
    total = 0
    for part in _step_parts(model):
        for linear in part.projections():
            total += _tensor_bytes(linear.weight) + _tensor_bytes(linear.bias)
        for vector in part.vectors():
            total += _tensor_bytes(vector)
    return total


def kv_bytes_per_token(model) -> int:
    """Bytes of keys and values one cached token takes over all layers."""
    kv, _, source = model.cache_needs()
    width = torch.empty((), dtype=model.dtype).element_size()
    return sum(2 * need.kv_heads * need.head_dim * width for need, src in zip(kv, source) if need is not None and src is None)


def kv_read_bytes_per_token(model) -> int:
    """Bytes of keys and values a decode step reads per cached token: every run that attends reads
    them, also one that reads another run's cache."""
    kv, _, _ = model.cache_needs()
    width = torch.empty((), dtype=model.dtype).element_size()
    return sum(2 * need.kv_heads * need.head_dim * width for need in kv if need is not None)


def linear_flops_per_token(model) -> int:
    """Multiply-adds times two of all projections for one token (the head excluded)."""
    total = 0
    for run in model.spec.schedule:
        for part in model.layers[run.layer].parts.values():
            for linear in part.projections():
                total += 2 * linear.out_features * linear.in_features
    return total


def attention_flops(model, tokens: int) -> float:
    """Causal attention of one sequence of ``tokens`` tokens: QK^T and PV over t(t+1)/2 pairs."""
    flops = 0.0
    kv, _, _ = model.cache_needs()
    for index, run in enumerate(model.spec.schedule):
        for user, mixer in zip(model.users[index], model.layers[run.layer].mixers()):
            if kv[user] is not None:
                flops += 2.0 * 2.0 * (tokens * (tokens + 1) / 2) * kv[user].head_dim * getattr(mixer, "heads", kv[user].kv_heads)
    return flops


def prefill_flops(model, tokens: int) -> float:
    """Projections for every token, causal attention, and the head at one position."""
    return float(linear_flops_per_token(model)) * tokens + attention_flops(model, tokens) + 2.0 * model.spec.vocab_size * model.spec.hidden_size


def measure_prefill(runtime, prompt, repeats: int = 3, warmup: int = 2) -> dict:
    """Whole prompts in one step, logits at each one's last position.  ``prompt`` is one list of
    token ids or a list of them (a batch of prompts of any lengths, packed into the one step)."""
    prompts = [prompt] if prompt and isinstance(prompt[0], int) else [list(p) for p in prompt]
    total = sum(len(p) for p in prompts)
    room = sum(-(-(len(p) + 1) // 64) * 64 for p in prompts)
    engine = runtime.new_engine(max_tokens=room, max_sequences=len(prompts), max_step_tokens=8192)
    times = []
    for i in range(warmup + repeats):
        slots = [engine.open() for _ in prompts]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([Entry(slot, p, [len(p) - 1]) for slot, p in zip(slots, prompts)])
        stop.record()
        torch.cuda.synchronize()
        for slot in slots:
            engine.close(slot)
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    engine.check_status()
    ms = sum(times) / len(times)
    model = runtime.model
    flops = (float(linear_flops_per_token(model)) * total + sum(attention_flops(model, len(p)) for p in prompts)
             + 2.0 * model.spec.vocab_size * model.spec.hidden_size * len(prompts))
    return {"ms": ms, "tokens": total, "sequences": len(prompts), "tokens_per_s": total / (ms / 1e3), "flops": flops}


def roofline(decode: dict | None, prefill: dict | None, pk: dict) -> dict:
    """Achieved rates and their fractions of the peaks: a decode step against the copy bandwidth
    (the bytes it has to read: every weight once and the live sequences' cache), a prefill against
    the matrix-product rate."""
    out: dict = {"peaks": pk["source"]}
    if decode is not None:
        gbs = decode["bytes_per_step"] / (decode["ms_per_step"] / 1e3) / 1e9
        out["decode"] = {"bound": "hbm", "bytes_per_step": int(decode["bytes_per_step"]), "achieved_gbs": gbs, "peak_gbs": pk["hbm_gbs"],
                         "frac": gbs / pk["hbm_gbs"]}
    if prefill is not None:
        tflops = prefill["flops"] / (prefill["ms"] / 1e3) / 1e12
        out["prefill"] = {"bound": "tensor", "flops": prefill["flops"], "achieved_tflops": tflops, "peak_tflops": pk["bf16_tflops"],
                          "frac": tflops / pk["bf16_tflops"]}
    return out


def class_fractions(model, classes: dict, pk: dict, prefill_prompts: list[list[int]], batch: int, mean_context: float) -> dict:
    """The classes' times against their own bounds: a prefill's products and attention against the
    matrix-product rate (their FLOP), a decode step's products against the copy bandwidth (the weights)
    and its attention against it too (the cache it reads); the rest (norms, rotation, embedding,
    sampling) has no bound worth naming and is given as time alone.  Times are those of kernels run
    one after another (see :func:`measure_classes`)."""
    def split(spans: dict) -> dict:
        out = {"products": 0.0, "attention": 0.0, "rest": 0.0}
        for name, entry in spans.items():
            kind = "products" if name.startswith("tt_gemm") else "attention" if name.startswith("tt_attention") else "rest"
            out[kind] += entry["ms"]
        return out

    tokens = sum(len(p) for p in prefill_prompts)
    prefill, decode = split(classes["prefill_step"]), split(classes["decode_step"])
    linear = float(linear_flops_per_token(model)) * tokens + 2.0 * model.spec.vocab_size * model.spec.hidden_size * len(prefill_prompts)
    attention = sum(attention_flops(model, len(p)) for p in prefill_prompts)
    peak_flops, peak_bytes = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    frac = lambda amount, ms, peak: round(amount / (ms / 1e3) / peak, 4) if ms > 0 else None
    return {
        "prefill": {"tokens": tokens, "products_ms": round(prefill["products"], 4), "products_frac": frac(linear, prefill["products"], peak_flops),
                    "attention_ms": round(prefill["attention"], 4), "attention_frac": frac(attention, prefill["attention"], peak_flops),
                    "rest_ms": round(prefill["rest"], 4)},
        "decode": {"batch": batch, "products_ms": round(decode["products"], 4),
                   "products_frac": frac(weight_bytes_per_step(model), decode["products"], peak_bytes),
                   "attention_ms": round(decode["attention"], 4),
                   "attention_frac": frac(kv_read_bytes_per_token(model) * mean_context * batch, decode["attention"], peak_bytes),
                   "rest_ms": round(decode["rest"], 4)},
        "how": "CUDA events around every kernel, kernels run one after another (no overlap between them)",
    }


def measure_classes(runtime, prompts: list[list[int]], context: int, prefill_prompts: list[list[int]] | None = None) -> dict:
    """Where the time of one prefill step and of one decode step goes, by class of kernel: both are
    run eagerly with every kernel call bracketed by CUDA events (:class:`~thintensor_b200.kernels.api.ClassTimer`).
    The kernels then run one after another without overlapping, so the sums are larger than the
    steps' real durations; the shares are what to read."""
    batch = len(prompts)
    per_sequence = -(-context // 64) * 64
    engine = runtime.new_engine(max_tokens=per_sequence * batch, max_sequences=batch)
    backend = EngineBackend(engine, SamplingParams(), use_graph=False)
    backend.start_batch(list(range(batch)), prompts, [context] * batch)          # compiles and sizes scratch memory
    state = backend._state_for(list(range(batch)))
    state.step(backend.params, False)
    with api.timed_classes() as timer:
        state.step(backend.params, False)
    decode = timer.summary()
    for position in range(batch):
        backend.finish(position)
    prefill_prompts = prompts if prefill_prompts is None else prefill_prompts
    slots = [engine.open() for _ in prefill_prompts]                 # once untimed: compiles and sizes what this shape needs
    engine.step([Entry(slot, p, [len(p) - 1]) for slot, p in zip(slots, prefill_prompts)])
    for slot in slots:
        engine.close(slot)
    engine.use_step_graphs = False                                    # the timed step runs kernel by kernel
    with api.timed_classes() as timer:
        slots = [engine.open() for _ in prefill_prompts]
        engine.step([Entry(slot, p, [len(p) - 1]) for slot, p in zip(slots, prefill_prompts)])
    prefill = timer.summary()
    for slot in slots:
        engine.close(slot)
    engine.check_status()
    return {"decode_step": decode, "prefill_step": prefill, "mean_context": sum(len(p) for p in prompts) / batch + 2,
            "decode_ms_serialised": sum(c["ms"] for c in decode.values()), "prefill_ms_serialised": sum(c["ms"] for c in prefill.values())}


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
    bytes_per_step = weight_bytes_per_step(runtime.model) + kv_read_bytes_per_token(runtime.model) * mean_context * batch
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

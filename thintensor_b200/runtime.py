"""The Python entry point: a model folder in, a runtime that steps and generates out.

    runtime = thintensor_b200.load_model("path/to/model", dtype="bf16")
    tokens = runtime.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)

The reference's usage is ``ThinGpuWeights(path, device, dtype)`` ->
``PagedKVCache(...)`` -> ``ThinGpuCausalLMRuntime(weights, kv_cache=cache)`` ->
``forward_token`` / ``logits`` / ``next_token_tensor`` (thinruntime/__init__.py:14-39,
thinruntime/gpu_runtime.py:12737-12774); option names (``dtype``, ``device``,
``context``, ``max_new_tokens``, ``temperature``, ``top_p``, ``top_k``, ``seed``) are
those of its command line (thinruntime/cli.py:165-264).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Sequence

import torch

from .cache.cache import BLOCK_TOKENS
from .config.base import read_config_json
from .config.registry import load_config
from .engine.engine import Engine
from .engine.generate import EngineBackend, GenerationStats, run_generation
from .engine.model import DecoderModel
from .sampling.sampler import SamplingParams
from .weights.loader import load_checkpoint
from .weights.random_init import write_model_folder

DTYPES = {
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, torch.bfloat16: torch.bfloat16,
    "fp32": torch.float32, "float32": torch.float32, torch.float32: torch.float32,
}


def parse_dtype(dtype) -> torch.dtype:
    if dtype not in DTYPES:
        raise ValueError(f"dtype must be bf16 (bfloat16) or fp32 (float32), got {dtype!r}")
    return DTYPES[dtype]


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"thintensor_b200 runs on a CUDA device only (asked for {device}); there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("thintensor_b200 needs a CUDA device and none is available; there is no CPU path")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def stop_ids_of(folder: Path | None, config) -> tuple[int, ...]:
    """End-of-sequence ids from generation_config.json and config.json, int or list, as
    the reference collects them (thinruntime/cli.py:4822-4888).  ``folder`` is None for a
    model that was not read from one."""
    ids = list(getattr(config, "eos_token_ids", ()))
    extra = None if folder is None else folder / "generation_config.json"
    if extra is not None and extra.is_file():
        eos = json.loads(extra.read_text(encoding="utf-8")).get("eos_token_id")
        if isinstance(eos, int):
            ids.append(eos)
        elif isinstance(eos, list):
            ids.extend(int(e) for e in eos)
    return tuple(dict.fromkeys(ids))


class Runtime:
    """A loaded model on one GPU."""

    def __init__(self, folder: Path | None, arch, config, model: DecoderModel):
        self.folder = folder
        self.architecture = arch
        self.config = config
        self.model = model
        self.stop_ids = stop_ids_of(folder, config)
        self._engine: Engine | None = None
        self._engine_key: tuple[int, int] | None = None

    def new_engine(self, max_tokens: int, max_sequences: int = 64, max_step_tokens: int = 8192, step_graphs: bool = True) -> Engine:
        """An engine whose cache holds ``max_tokens`` tokens (each sequence's count
        rounded up to whole blocks of 64) for up to ``max_sequences`` live sequences.
        ``step_graphs``: whether steps of a shape that has run before are replayed from a CUDA graph."""
        blocks = max(1, -(-int(max_tokens) // BLOCK_TOKENS))
        cache = self.model.new_cache(blocks, max_sequences)
        return Engine(self.model, cache, max_step_tokens, step_graphs)

    def engine_for(self, max_tokens: int, max_sequences: int) -> Engine:
        """The runtime's own engine, kept from call to call (with its cache, its scratch memory and
        the decode steps it has captured) as long as it is large enough; a call that needs more
        replaces it with a larger one."""
        have = self._engine_key
        if self._engine is None or have[0] < max_tokens or have[1] < max_sequences:
            key = (max(max_tokens, have[0] if have else 0), max(max_sequences, have[1] if have else 0))
            self._engine = None                                    # the old cache goes before the new one comes
            self._engine = self.new_engine(*key)
            self._engine_key = key
        return self._engine

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 200, temperature: float = 0.0, top_p: float = 1.0,
                 top_k: int = 0, seed: int = 0, stop_ids: Sequence[int] | None = None, context: int | None = None,
                 batch_size: int = 8, use_graph: bool = True, stats: GenerationStats | None = None) -> list[list[int]]:
        """New tokens for every prompt (lists of token ids).  ``stop_ids`` default to the
        model's end-of-sequence ids; pass ``()`` to always generate ``max_new_tokens``."""
        prompts = [list(p) for p in prompts]
        stops = self.stop_ids if stop_ids is None else tuple(stop_ids)
        longest = max((len(p) for p in prompts), default=0) + max_new_tokens
        per_sequence = -(-longest // BLOCK_TOKENS) * BLOCK_TOKENS
        live = min(batch_size, max(1, len(prompts)))
        engine = self.engine_for(per_sequence * live, live)
        backend = EngineBackend(engine, SamplingParams(temperature, top_k, top_p, seed), use_graph)
        return run_generation(backend, prompts, max_new_tokens, stops, batch_size, context, stats)


def load_model(path: str | Path, dtype="bf16", device="cuda") -> Runtime:
    """Read ``config.json`` and the safetensors of a model folder and put the model on
    the GPU.  The model class is chosen by config.json through the architecture registry."""
    folder = Path(path)
    torch_dtype = parse_dtype(dtype)
    device = require_cuda(device)
    arch, config = load_config(folder)
    model = DecoderModel(arch.describe(config), torch_dtype, device)
    wrapped = isinstance(read_config_json(folder).get("text_config"), dict)    # a multimodal wrapper's folder
    model.bind(load_checkpoint(folder, model.weight_declarations(), torch_dtype, device, wrapped))
    return Runtime(folder, arch, config, model)


def save_random_model(folder: str | Path, config, seed: int = 0, dtype: str = "bfloat16") -> Path:
    """Write a model folder (config.json, model.safetensors) with random weights for a
    typed configuration or a config.json dict."""
    if isinstance(config, dict):
        arch, config = load_config(config)
    else:
        arch, _ = load_config(config.to_dict())
    declared = DecoderModel(arch.describe(config), torch.float32, None).weight_declarations()
    return write_model_folder(folder, config, declared, seed, dtype)


def random_model(config, seed: int = 0, dtype="bf16", device="cuda") -> Runtime:
    """A runtime whose weights are drawn on the device (N(0, 0.02), norm weights
    1 + N(0, 0.1)) without writing a folder: for benchmarks at sizes whose files would
    take minutes to write.  ``config`` is a config.json dict or a typed configuration.

    The numbers are NOT those :func:`save_random_model` writes for the same seed: this function
    draws with the device's generator, that one with the host's, tensor by tensor in the same order.
    Use a written folder wherever another implementation has to see the same weights."""
    torch_dtype = parse_dtype(dtype)
    device = require_cuda(device)
    arch, config = load_config(config if isinstance(config, dict) else config.to_dict())
    model = DecoderModel(arch.describe(config), torch_dtype, device)
    generator = torch.Generator(device=device)
    generator.manual_seed(int(seed))
    tensors: dict[str, torch.Tensor] = {}
    for name, decl in model.weight_declarations().items():
        if decl.alias_of is not None and decl.prefer_alias:
            continue
        if decl.integer:
            tensors[name] = torch.zeros(decl.shape, dtype=torch.int32, device=device)
            continue
        noise = torch.randn(decl.shape, generator=generator, device=device, dtype=torch.float32)
        value = 1.0 + 0.1 * noise if decl.init == "norm" else (noise * 0.02 if decl.init == "normal" else noise * 0.0)
        tensors[name] = value.to(torch_dtype)
        del noise, value
    model.bind(tensors)
    return Runtime(None, arch, config, model)

"""The reference arm of bench.py: random-unknown-username/Thintensor itself, unmodified, as
installed offline into ``baseline/_ref``, on the same model shape and workload.

Nothing of this repository's engine is on this path.  The reference loads only its own
``.thin`` archives, which its Rust converter makes; that converter cannot be built here
(no cargo), so the archive is written by the few lines below from the layout its reader
documents (thinruntime/archive.py:9-13, 99-208): an 88-byte header, a JSON manifest, a
page table, raw bfloat16 pages.  From there on everything is the reference's public
API and stock code path, exactly as its own ``benchmark_gpu_runtime`` uses them
(thinruntime/gpu_runtime.py:12719-12760): ``ThinGpuWeights`` -> ``PagedKVCache`` ->
``ThinGpuCausalLMRuntime(weights, kv_cache=cache)`` -> ``forward_token`` /
``next_token_tensor``.

The reference runs one sequence, one token per call (its results carry ``batch_size: 1``,
scripts/thin_runtime.py:1115-1117) and feeds a prompt token by token
(thinruntime/cli.py:2802-2807).  A batch of 8 is therefore served the only way it can
be: one sequence after the other, each with its 2,048-token prompt; the reported value is
all decoded tokens divided by all decode time.  If that would take longer than the time
limit, fewer of the 8 sequences are run and the line says how many.
"""
from __future__ import annotations

import hashlib
import json
import struct
import sys
import tempfile
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def write_thin(path: Path, shape: dict, seed: int) -> None:
    """A bfloat16 ``.thin`` archive of random weights (N(0, 0.02), norms 1 + N(0, 0.1))."""
    import torch

    g = torch.Generator().manual_seed(seed)
    hidden, layers = shape["hidden_size"], shape["num_hidden_layers"]
    heads, kv_heads, head_dim = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"]
    inter, vocab = shape["intermediate_size"], shape["vocab_size"]
    specs = [("model.embed_tokens.weight", (vocab, hidden), "normal")]
    for layer in range(layers):
        p = f"model.layers.{layer}."
        specs += [
            (p + "input_layernorm.weight", (hidden,), "norm"),
            (p + "self_attn.q_proj.weight", (heads * head_dim, hidden), "normal"),
            (p + "self_attn.k_proj.weight", (kv_heads * head_dim, hidden), "normal"),
            (p + "self_attn.v_proj.weight", (kv_heads * head_dim, hidden), "normal"),
            (p + "self_attn.o_proj.weight", (hidden, heads * head_dim), "normal"),
            (p + "post_attention_layernorm.weight", (hidden,), "norm"),
            (p + "mlp.gate_proj.weight", (inter, hidden), "normal"),
            (p + "mlp.up_proj.weight", (inter, hidden), "normal"),
            (p + "mlp.down_proj.weight", (hidden, inter), "normal"),
        ]
    specs.append(("model.norm.weight", (hidden,), "norm"))
    scaling = shape["rope_scaling"]
    model = {
        "model_type": "llama", "arch": "LlamaForCausalLM", "hidden_size": hidden, "layers": layers, "heads": heads,
        "kv_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter, "vocab_size": vocab,
        "rms_norm_eps": shape["rms_norm_eps"], "norm_eps": shape["rms_norm_eps"], "norm_kind": "rms_norm",
        "rope_theta": shape["rope_theta"], "tie_word_embeddings": True, "activation": "silu",
        "max_position_embeddings": shape["max_position_embeddings"], "rope_variant": "llama3", "rope_scaling": scaling,
        "rope_parameters": dict(scaling, rope_theta=shape["rope_theta"]),
        "original_max_position_embeddings": scaling["original_max_position_embeddings"],
    }
    pages = []
    for name, dims, _ in specs:
        count = 1
        for d in dims:
            count *= d
        layer = int(name.split(".")[2]) if name.startswith("model.layers.") else None
        pages.append({"id": name, "kind": "tensor", "layer": layer, "op": name.rsplit(".", 2)[-2], "dtype": "BF16",
                      "shape": list(dims), "backend_layout": "row_major", "size": count * 2,
                      "checksum": hashlib.sha256(name.encode()).hexdigest()})      # distinct per page: equal checksums would alias pages
    manifest = json.dumps({"format": "thin", "version": 0, "model": model, "execution_tape": [], "pages": pages, "memory_plan": {}}).encode()
    tail = struct.calcsize("<QQQI32s")
    table_len = sum(2 + len(p["id"].encode()) + tail for p in pages)
    table_off = 88 + len(manifest)
    data_off = table_off + table_len
    table, offset = b"", data_off
    for page in pages:
        ident = page["id"].encode()
        table += struct.pack("<H", len(ident)) + ident + struct.pack("<QQQI32s", offset, page["size"], page["size"], 0, bytes(32))
        offset += page["size"]
    with path.open("wb") as out:
        out.write(struct.pack("<8sIIQQQQQ32s", b"THINv0\0\0", 88, 0, 88, len(manifest), table_off, len(pages), data_off, bytes(32)))
        out.write(manifest)
        out.write(table)
        for name, dims, kind in specs:
            noise = torch.randn(dims, generator=g)
            value = (1.0 + 0.1 * noise) if kind == "norm" else 0.02 * noise
            out.write(value.to(torch.bfloat16).view(torch.int16).numpy().tobytes())


def run(shape: dict, metric: str, batch: int, prompt_len: int, context: int, steps: int, warmup: int, limit_s: float = 150.0) -> dict:
    if not (REF / "thinruntime").is_dir():
        return {"impl": "reference", "unavailable": f"the reference is not installed under {REF} (pip install --target baseline/_ref was not run here)"}
    sys.path.insert(0, str(REF))
    import torch
    from thinruntime.gpu_runtime import PagedKVCache, ThinGpuCausalLMRuntime, ThinGpuWeights

    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, shape["vocab_size"], (prompt_len,), generator=g).tolist() for _ in range(batch)]
    with tempfile.TemporaryDirectory() as folder:
        archive = Path(folder) / "model.thin"
        write_thin(archive, shape, seed=0)
        weights = ThinGpuWeights(archive, device="cuda", dtype=torch.bfloat16)
        cache = PagedKVCache(layers=shape["num_hidden_layers"], kv_heads=shape["num_key_value_heads"], head_dim=shape["head_dim"],
                             device=weights.device, dtype=torch.bfloat16, old_codec="bf16")
        runtime = ThinGpuCausalLMRuntime(weights, kv_cache=cache)
        decoded, decode_ms, prefill_s, sequences_run = 0, 0.0, 0.0, 0
        started = time.perf_counter()
        for prompt in prompts:
            if sequences_run and (time.perf_counter() - started) * (sequences_run + 1) / sequences_run > limit_s:
                break
            cache.reset(reuse_pages=True)
            clock = time.perf_counter()
            hidden = None
            for index, token in enumerate(prompt):                    # the reference's prefill: token by token
                hidden = runtime.forward_token(token, token_index=index)
            runtime.begin_decode(len(prompt))
            torch.cuda.synchronize()
            prefill_s += time.perf_counter() - clock
            position = len(prompt)
            for _ in range(warmup):
                token = runtime.next_token_tensor(hidden)
                hidden = runtime.forward_token(token, token_index=position)
                position += 1
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):                                     # ids stay on the device, as in scripts/thin_runtime.py:981-1011
                token = runtime.next_token_tensor(hidden)
                hidden = runtime.forward_token(token, token_index=position)
                position += 1
            stop.record()
            torch.cuda.synchronize()
            decode_ms += start.elapsed_time(stop)
            decoded += steps
            sequences_run += 1
        weights.close()
    value = decoded / (decode_ms / 1e3)
    return {
        "impl": "reference", "metric": metric, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(decode_ms / decoded * batch, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) from a seed, token ids uniform in [0, vocab)",
        "config": {"model": "Llama-3.2-1B shape", "layers": shape["num_hidden_layers"], "global_batch": batch, "prompt_len": prompt_len,
                   "seq_len": context, "served": "one sequence at a time (the engine has no batching)", "sequences_run": sequences_run,
                   "prefill": "token by token", "prefill_tokens_per_s": round(prompt_len * sequences_run / prefill_s, 1)},
    }

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

import sys
import tempfile
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def write_random_archive(path: Path, shape: dict, seed: int) -> None:
    """A bfloat16 ``.thin`` archive of random weights (N(0, 0.02), norms 1 + N(0, 0.1))."""
    import torch

    from thin_archive import llama_manifest_model, write_thin

    g = torch.Generator().manual_seed(seed)
    hidden, layers = shape["hidden_size"], shape["num_hidden_layers"]
    heads, kv_heads, head_dim = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"]
    inter, vocab = shape["intermediate_size"], shape["vocab_size"]
    specs = [("model.embed_tokens.weight", (vocab, hidden))]
    for layer in range(layers):
        p = f"model.layers.{layer}."
        specs += [
            (p + "input_layernorm.weight", (hidden,)),
            (p + "self_attn.q_proj.weight", (heads * head_dim, hidden)),
            (p + "self_attn.k_proj.weight", (kv_heads * head_dim, hidden)),
            (p + "self_attn.v_proj.weight", (kv_heads * head_dim, hidden)),
            (p + "self_attn.o_proj.weight", (hidden, heads * head_dim)),
            (p + "post_attention_layernorm.weight", (hidden,)),
            (p + "mlp.gate_proj.weight", (inter, hidden)),
            (p + "mlp.up_proj.weight", (inter, hidden)),
            (p + "mlp.down_proj.weight", (hidden, inter)),
        ]
    specs.append(("model.norm.weight", (hidden,)))
    model = llama_manifest_model(hidden=hidden, layers=layers, heads=heads, kv_heads=kv_heads, head_dim=head_dim, inter=inter, vocab=vocab,
                                 eps=shape["rms_norm_eps"], theta=shape["rope_theta"], tied=True,
                                 max_pos=shape["max_position_embeddings"], scaling=shape["rope_scaling"])

    def draw(name, dims):
        noise = torch.randn(dims, generator=g)
        return (1.0 + 0.1 * noise) if name.endswith("norm.weight") else 0.02 * noise

    write_thin(path, model, specs, "BF16", draw)


def run(shape: dict, metric: str, batch: int, prompt_len: int, context: int, steps: int, warmup: int, limit_s: float = 150.0) -> dict:
    if not (REF / "thinruntime").is_dir():
        return {"impl": "reference", "unavailable": f"the reference is not installed under {REF} (pip install --target baseline/_ref was not run here)"}
    sys.path.insert(0, str(REF))
    sys.path.insert(0, str(HERE))
    import torch
    from thinruntime.gpu_runtime import PagedKVCache, ThinGpuCausalLMRuntime, ThinGpuWeights

    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, shape["vocab_size"], (prompt_len,), generator=g).tolist() for _ in range(batch)]
    with tempfile.TemporaryDirectory() as folder:
        archive = Path(folder) / "model.thin"
        write_random_archive(archive, shape, seed=0)
        weights = ThinGpuWeights(archive, device="cuda", dtype=torch.bfloat16)
        cache = PagedKVCache(layers=shape["num_hidden_layers"], kv_heads=shape["num_key_value_heads"], head_dim=shape["head_dim"],
                             device=weights.device, dtype=torch.bfloat16, old_codec="bf16")
        runtime = ThinGpuCausalLMRuntime(weights, kv_cache=cache)
        decoded, decode_ms, prefill_s, sequences_run = 0, 0.0, 0.0, 0
        e2e_decoded, e2e_s, e2e_d2h = 0, 0.0, 8
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
            # end to end, the way the reference's own `run` command decodes (thinruntime/cli.py:2826-2858):
            # next_token_tensor -> synchronize -> .item() on the host -> forward_token(int)
            e2e_steps = min(steps, context - position - 1)
            clock = time.perf_counter()
            for _ in range(e2e_steps):
                token_tensor = runtime.next_token_tensor(hidden)
                torch.cuda.synchronize()
                token = int(token_tensor.item())
                e2e_d2h = token_tensor.element_size()
                hidden = runtime.forward_token(token, token_index=position)
                position += 1
            torch.cuda.synchronize()
            e2e_s += time.perf_counter() - clock
            e2e_decoded += e2e_steps
        weights.close()
    value = decoded / (decode_ms / 1e3)
    return {
        "impl": "reference", "metric": metric, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(decode_ms / decoded * batch, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) from a seed, token ids uniform in [0, vocab)",
        "config": {"model": "Llama-3.2-1B shape", "layers": shape["num_hidden_layers"], "global_batch": batch, "prompt_len": prompt_len,
                   "seq_len": context, "served": "one sequence at a time (the engine has no batching)", "sequences_run": sequences_run,
                   "prefill": "token by token", "prefill_tokens_per_s": round(prompt_len * sequences_run / prefill_s, 1)},
        # the reference's own generation loop: one host read of the token per step, the id handed back as a Python int
        "e2e": {"value": round(e2e_decoded / e2e_s, 1) if e2e_s > 0 else None, "unit": "tokens/s", "steps": e2e_decoded,
                "h2d_bytes_per_step": 8, "d2h_bytes_per_step": e2e_d2h,
                "how": "next_token_tensor, synchronize, .item(), forward_token(int) per token, as thinruntime/cli.py:2826-2858"},
        # the engine serves one sequence at a time, so its value is also its rate at batch 1
        "points": {"decode_b1": round(value, 1)},
    }

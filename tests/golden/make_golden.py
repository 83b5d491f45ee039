"""Make tests/golden/reference_logits.npz: logits of random-unknown-username/Thintensor's
OWN runtime, on the CPU, for three tiny random Llama models.

Run once, by hand, from the repository root, with the reference checkout on the path:

    PYTHONPATH=/path/to/Thintensor python tests/golden/make_golden.py

What it does.  For each tiny configuration (tiny A, B and F of tests/conftest.py) it draws
weights from a seeded CPU generator (function ``golden_weights`` below, which
tests/test_plain.py imports so that the oracle gets the very same numbers), writes them
as a float32 ``.thin`` archive in a temporary folder (the archive layout is read off
thinruntime/archive.py:9-13, 99-208: an 88-byte header, a JSON manifest, a page table,
the raw pages), opens it with the reference's ``ThinGpuWeights`` / ``PagedKVCache`` /
``ThinGpuCausalLMRuntime`` on ``device="cpu"`` with its PyTorch kernels, feeds each
prompt token by token through ``forward_token`` (its only mode) and records
``logits(hidden)`` at every position.  tests/test_plain.py compares the plain
implementation with these numbers.  Nothing of the reference's code is copied; it is
imported and called.  The reference needs the installed ``transformers`` package for
the llama3 frequency scaling, which it calls as a black box.
"""
from __future__ import annotations

import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

CONFIGS = {
    "a": {"layers": 2, "hidden": 64, "heads": 4, "kv_heads": 2, "head_dim": 16, "inter": 128, "vocab": 256,
          "theta": 10000.0, "eps": 1e-5, "tied": True, "scaling": None, "max_pos": 2048, "seed": 0},
    "b": {"layers": 3, "hidden": 96, "heads": 3, "kv_heads": 1, "head_dim": 32, "inter": 320, "vocab": 512,
          "theta": 500000.0, "eps": 1e-6, "tied": False, "max_pos": 512, "seed": 2,
          "scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                      "original_max_position_embeddings": 64}},
    # biases on every projection (the reference adds them where the tensors exist), one key/value head per query head
    "f": {"layers": 2, "hidden": 80, "heads": 5, "kv_heads": 5, "head_dim": 16, "inter": 112, "vocab": 199,
          "theta": 20000.0, "eps": 2e-5, "tied": True, "scaling": None, "max_pos": 1024, "seed": 9, "bias": True},
}
PROMPTS = {"a": [(5, 11), (9, 12), (2, 13)], "b": [(17, 21), (1, 22), (40, 23), (70, 24)], "f": [(6, 31), (23, 32)]}   # (length, seed)


def prompt_tokens(vocab: int, length: int, seed: int) -> list[int]:
    return torch.randint(0, vocab, (length,), generator=torch.Generator().manual_seed(seed)).tolist()


def golden_weights(c: dict) -> dict[str, torch.Tensor]:
    """float32 weights by checkpoint name: matrices N(0, 0.02) (queries and keys times 8,
    tables times 20, so that attention is peaked and logits are of order one), norm
    weights 1 + N(0, 0.1); with ``bias`` every projection also gets a bias N(0, 0.2), drawn
    right after its matrix."""
    g = torch.Generator().manual_seed(c["seed"])

    def normal(*shape, scale=0.02):
        return torch.randn(*shape, generator=g) * scale

    q, kv = c["heads"] * c["head_dim"], c["kv_heads"] * c["head_dim"]
    w = {"model.embed_tokens.weight": normal(c["vocab"], c["hidden"], scale=0.4)}

    def projection(name, rows, cols, scale=0.02):
        w[name + ".weight"] = normal(rows, cols, scale=scale)
        if c.get("bias"):
            w[name + ".bias"] = normal(rows, scale=0.2)

    for layer in range(c["layers"]):
        p = f"model.layers.{layer}."
        w[p + "input_layernorm.weight"] = 1.0 + normal(c["hidden"], scale=0.1)
        projection(p + "self_attn.q_proj", q, c["hidden"], 0.16)
        projection(p + "self_attn.k_proj", kv, c["hidden"], 0.16)
        projection(p + "self_attn.v_proj", kv, c["hidden"])
        projection(p + "self_attn.o_proj", c["hidden"], q)
        w[p + "post_attention_layernorm.weight"] = 1.0 + normal(c["hidden"], scale=0.1)
        projection(p + "mlp.gate_proj", c["inter"], c["hidden"])
        projection(p + "mlp.up_proj", c["inter"], c["hidden"])
        projection(p + "mlp.down_proj", c["hidden"], c["inter"])
    w["model.norm.weight"] = 1.0 + normal(c["hidden"], scale=0.1)
    if not c["tied"]:
        w["lm_head.weight"] = normal(c["vocab"], c["hidden"], scale=0.4)
    return w


def write_thin(path: Path, c: dict, weights: dict[str, torch.Tensor]) -> None:
    """The weights as a float32 archive, through the one archive writer this repository has
    (baseline/thin_archive.py, shared with the benchmark's reference arm)."""
    sys.path.insert(0, str(HERE.parent.parent / "baseline"))
    from thin_archive import llama_manifest_model, write_thin as write_archive

    model = llama_manifest_model(hidden=c["hidden"], layers=c["layers"], heads=c["heads"], kv_heads=c["kv_heads"], head_dim=c["head_dim"],
                                 inter=c["inter"], vocab=c["vocab"], eps=c["eps"], theta=c["theta"], tied=c["tied"], max_pos=c["max_pos"],
                                 scaling=c["scaling"], bias=bool(c.get("bias")))
    write_archive(path, model, [(name, tuple(t.shape)) for name, t in weights.items()], "F32", lambda name, shape: weights[name])


def reference_logits(archive: Path, c: dict, tokens: list[int]) -> np.ndarray:
    from thinruntime.gpu_runtime import PagedKVCache, ThinGpuCausalLMRuntime, ThinGpuWeights

    weights = ThinGpuWeights(archive, device="cpu", dtype=torch.float32)
    cache = PagedKVCache(c["layers"], c["kv_heads"], c["head_dim"], device="cpu", dtype=torch.float32, policy="full")
    runtime = ThinGpuCausalLMRuntime(weights, kv_cache=cache, kernel_backend="torch", attention_backend="torch", exact_hf_mode=True)
    rows = []
    for index, token in enumerate(tokens):
        hidden = runtime.forward_token(int(token), token_index=index)
        rows.append(runtime.logits(hidden).float().numpy().copy())
    return np.stack(rows)


def main() -> None:
    out = {}
    with tempfile.TemporaryDirectory() as folder:
        for name, c in CONFIGS.items():
            archive = Path(folder) / f"tiny_{name}.thin"
            write_thin(archive, c, golden_weights(c))
            for index, (length, seed) in enumerate(PROMPTS[name]):
                tokens = prompt_tokens(c["vocab"], length, seed)
                logits = reference_logits(archive, c, tokens)
                # keep the file small: every position of short prompts, the last 8 of long ones
                out[f"{name}_{index}"] = logits[-8:].astype(np.float32)
                print(name, index, logits.shape, float(np.abs(logits).max()))
    np.savez_compressed(HERE / "reference_logits.npz", **out)
    print("wrote", HERE / "reference_logits.npz")


if __name__ == "__main__":
    main()

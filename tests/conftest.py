"""Shared fixtures: tiny configurations, model folders with random weights, and the
plain implementation's outputs for them."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations that differ in every size and option, and a third whose sizes
# are no powers of two anywhere (head size 48, odd vocabulary).
TINY = {
    "a": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
        "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": True, "max_position_embeddings": 2048, "eos_token_id": 7,
    },
    "b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
        "intermediate_size": 320, "vocab_size": 512, "rope_theta": 500000.0, "rms_norm_eps": 1e-6,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "max_position_embeddings": 512, "tie_word_embeddings": False, "eos_token_id": [3, 11],
    },
    "c": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 2, "hidden_size": 144, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
        "intermediate_size": 200, "vocab_size": 311, "rope_theta": 250000.0, "rms_norm_eps": 3e-6,
        "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 2.0, "high_freq_factor": 8.0,
                         "original_max_position_embeddings": 128},
        "max_position_embeddings": 1024, "tie_word_embeddings": True,
    },
    # head sizes 64 and 128, the sizes the tcgen05 prompt attention and the pipelined decode attention take
    "d": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
        "intermediate_size": 192, "vocab_size": 300, "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
        "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "max_position_embeddings": 4096, "tie_word_embeddings": True,
    },
    "e": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 2, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 128,
        "intermediate_size": 160, "vocab_size": 257, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
        "max_position_embeddings": 4096, "tie_word_embeddings": False,
    },
    # the options no checkpoint of the family switches on: biases on every projection; one key/value head per query head
    "f": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 16,
        "intermediate_size": 112, "vocab_size": 199, "rope_theta": 20000.0, "rms_norm_eps": 2e-5,
        "attention_bias": True, "mlp_bias": True, "max_position_embeddings": 1024, "tie_word_embeddings": True,
    },
}
SEEDS = {"a": 0, "b": 2, "c": 5, "d": 7, "e": 8, "f": 9}


def write_tiny_model(folder: Path, name: str, stored: str = "float32", sharpen: float = 8.0) -> Path:
    """A model folder for tiny configuration ``name``.  The query and key projections
    are scaled by ``sharpen`` so that attention is far from uniform: a wrong key, a key
    of another sequence or a missing far key then moves the logits by much more than
    any tolerance."""
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.weights.random_init import STORED_DTYPES, random_tensors
    from thintensor_b200.weights.safetensors_io import write_safetensors

    arch, config = load_config(TINY[name])
    declared = DecoderModel(arch.describe(config), torch.float32, None).weight_declarations()
    tensors = random_tensors(declared, SEEDS[name], torch.float32)
    for key in tensors:
        if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
            tensors[key] = tensors[key] * sharpen
        elif key.endswith("embed_tokens.weight") or key.endswith("lm_head.weight"):
            tensors[key] = tensors[key] * 20.0          # hidden states and logits of order one
        elif key.endswith(".bias"):
            tensors[key] = tensors[key] * 10.0          # a bias that is dropped or put on the wrong rows shows
    tensors = {k: v.to(STORED_DTYPES[stored]) if v.is_floating_point() else v for k, v in tensors.items()}
    folder.mkdir(parents=True, exist_ok=True)
    raw = dict(TINY[name])
    raw["torch_dtype"] = stored
    (folder / "config.json").write_text(json.dumps(raw, indent=2))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name, stored dtype -> folder; made once per session in a temporary folder."""
    base = tmp_path_factory.mktemp("models")
    made: dict[tuple[str, str], Path] = {}

    def get(name: str, stored: str = "float32") -> Path:
        key = (name, stored)
        if key not in made:
            made[key] = write_tiny_model(base / f"{name}-{stored}", name, stored)
        return made[key]

    return get


def token_ids(vocab: int, length: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


_oracle_cache: dict = {}


def oracle_logits(folder: Path, tokens: list[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the plain implementation for one whole sequence."""
    import plain_llama

    key = (str(folder), tuple(tokens))
    if key not in _oracle_cache:
        model_key = ("model", str(folder))
        if model_key not in _oracle_cache:
            _oracle_cache[model_key] = plain_llama.read_model(folder)
        cfg, weights = _oracle_cache[model_key]
        _oracle_cache[key] = plain_llama.forward(cfg, weights, tokens)
    return _oracle_cache[key]


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    """float32: every logit within 2e-4 of the oracle, relative to the largest logit.
    bfloat16: the reference's ``exact_pass`` measures (cosine >= 0.999 per position,
    scripts/compare_hf_thin_logits.py:2026-2037) and a bound on the largest error."""
    got = got.double().cpu()
    want = want.double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    if dtype == "float32":
        assert err <= 2e-4 * scale, f"{what}: max |diff| {err:.3e} with logits up to {scale:.3f}"
    else:
        cos = torch.nn.functional.cosine_similarity(got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1]), dim=-1)
        assert float(cos.min()) >= 0.999, f"{what}: cosine {float(cos.min()):.5f}"
        assert err <= 0.06 * scale, f"{what}: max |diff| {err:.3e} with logits up to {scale:.3f}"

"""Layers of the real sizes (Llama-3.2-1B, 3.2-3B and 3.1-8B layer shapes, two layers,
a shortened vocabulary) against the plain implementation: a prompt long enough for
tensor-core tiles in every projection, then decoding, in bfloat16; and the float32 path
of the 1B shape.  These are the sizes at which head size 128, groups of 3 and 4 query
heads per key/value head, k = 14336 and split k-slices are exercised for real."""
from __future__ import annotations

import json

import pytest
import torch

import plain_llama
from conftest import assert_close, token_ids

pytestmark = pytest.mark.gpu

SHAPES = {
    "1b": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, factor=32.0, tied=True),
    "3b": dict(hidden_size=3072, num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192, factor=32.0, tied=True),
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, factor=8.0, tied=False),
}


def write_model(folder, shape, stored, layers=2, vocab=4099):
    import thintensor_b200
    from thintensor_b200.weights.safetensors_io import write_safetensors
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel

    s = SHAPES[shape]
    raw = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers, "vocab_size": vocab,
        "hidden_size": s["hidden_size"], "num_attention_heads": s["num_attention_heads"], "num_key_value_heads": s["num_key_value_heads"],
        "head_dim": s["head_dim"], "intermediate_size": s["intermediate_size"], "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
        "rope_scaling": {"rope_type": "llama3", "factor": s["factor"], "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "tie_word_embeddings": s["tied"], "max_position_embeddings": 131072,
    }
    arch, config = load_config(raw)
    declared = DecoderModel(arch.describe(config), torch.float32, None).weight_declarations()
    g = torch.Generator().manual_seed(11)
    tensors = {}
    for name, decl in declared.items():
        if decl.alias_of is not None and decl.prefer_alias:
            continue
        noise = torch.randn(decl.shape, generator=g)
        if decl.init == "norm":
            value = 1.0 + 0.1 * noise
        elif name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
            value = noise * 0.03        # scores a few units apart: attention is peaked, yet bfloat16 rounding of q and k does not reshuffle it
        elif "embed_tokens" in name or "lm_head" in name:
            value = noise * 0.3
        else:
            value = noise * 0.02
        tensors[name] = value.to(torch.bfloat16 if stored == "bfloat16" else torch.float32)
    folder.mkdir(parents=True, exist_ok=True)
    raw["torch_dtype"] = stored
    (folder / "config.json").write_text(json.dumps(raw))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


def plain_logits(folder, tokens, places):
    cfg, weights = plain_llama.read_model(folder)
    return plain_llama.forward(cfg, weights, tokens, dtype=torch.float32)[places].double()


@pytest.mark.parametrize("shape", ["1b", "3b", "8b"])
def test_bfloat16_real_layer_sizes(tmp_path, shape):
    import thintensor_b200
    from thintensor_b200.engine.engine import Entry

    folder = write_model(tmp_path / shape, shape, "bfloat16")
    runtime = thintensor_b200.load_model(folder, dtype="bf16")
    engine = runtime.new_engine(max_tokens=1024, max_sequences=3)
    tokens = token_ids(4099, 300, 31)
    other = token_ids(4099, 140, 32)
    places = [0, 100, 255, 256, 257, 270, 299]
    want = plain_logits(folder, tokens, places)
    # the prompt's first 258 tokens together with another sequence, then one token at a time
    a, b = engine.open(), engine.open()
    got = {}
    logits = engine.step([Entry(b, other[:130], []), Entry(a, tokens[:258], [0, 100, 255, 256, 257])])
    for row, place in enumerate([0, 100, 255, 256, 257]):
        got[place] = logits[row]
    for t in range(258, 300):
        logits = engine.step([Entry(a, [tokens[t]], [0]), Entry(b, [other[130 + (t - 258) % 10]], [])])
        got[t] = logits[0]
    engine.close(a)
    engine.close(b)
    engine.check_status()
    assert_close(torch.stack([got[p] for p in places]), want, "bfloat16", f"{shape} shape")


@pytest.mark.parametrize("shape", ["1b", "3b", "8b"])
def test_float32_real_layer_sizes(tmp_path, shape):
    """The true 32-bit path at the three layer sizes (two layers each): head sizes 64 and 128, groups of
    3 and 4 query heads, k = 8,192 and 14,336 through the exact product and the exact attention."""
    import thintensor_b200
    from thintensor_b200.engine.engine import Entry

    folder = write_model(tmp_path / "m", shape, "float32")
    runtime = thintensor_b200.load_model(folder, dtype="fp32")
    engine = runtime.new_engine(max_tokens=512, max_sequences=1)
    tokens = token_ids(4099, 150, 33)
    places = [0, 63, 64, 140, 149]
    want = plain_llama.forward(*plain_llama.read_model(folder), tokens, dtype=torch.float64)[places]
    slot = engine.open()
    got = {}
    logits = engine.step([Entry(slot, tokens[:141], [0, 63, 64, 140])])
    for row, place in enumerate([0, 63, 64, 140]):
        got[place] = logits[row]
    for t in range(141, 150):
        got[t] = engine.step([Entry(slot, [tokens[t]], [0])])[0]
    engine.close(slot)
    engine.check_status()
    assert_close(torch.stack([got[p] for p in places]), want, "float32", f"{shape} shape in float32")


def test_long_prompt_whole_and_in_pieces(tmp_path):
    """A 4,800-token prompt of the 1B layer sizes, whole (the output projections add their product into
    the residual stream inside the kernel) and in pieces of 1,024 tokens (their k is cut into slices and
    the norm kernel does the addition): the same logits."""
    import thintensor_b200
    from thintensor_b200.engine.engine import Entry
    from thintensor_b200.kernels import api

    folder = write_model(tmp_path / "m", "1b", "bfloat16")
    runtime = thintensor_b200.load_model(folder, dtype="bf16")
    tokens = token_ids(4099, 4800, 35)
    places = [0, 2047, 2048, 4095, 4700, 4799]
    assert api.gemm_tcgen05_accumulate_pays(4800, 2048, 2048) and not api.gemm_tcgen05_accumulate_pays(1024, 2048, 8192)
    results = []
    for piece in (8192, 1024):
        engine = runtime.new_engine(max_tokens=4864, max_sequences=1, max_step_tokens=piece)
        slot = engine.open()
        results.append(engine.step([Entry(slot, tokens, places)]).double().cpu())
        engine.close(slot)
        engine.check_status()
        if piece == 8192:
            # 19 x 8 = 152 tiles of 256 x 256 fill two thirds of three rounds of a B200's 74 CTA pairs: the pairs share the tiles' k,
            # which leaves their shares in the workspace and its flags zero
            shares = engine.workspace.get_zeroed("gemm.shares", (api.gemm_tcgen05_shares_words(),), torch.int32)
            flags = shares[-(shares.numel() // (32 * 256 + 1)):]
            assert int(flags.abs().sum().item()) == 0
            if api.sm_count() == 148:
                assert int(shares.abs().sum().item()) != 0
    assert_close(results[0], results[1], "bfloat16", "whole against pieces")
    # and the first positions against the plain implementation (the whole prompt would take it minutes)
    want = plain_logits(folder, tokens[:300], [0, 299])
    engine = runtime.new_engine(max_tokens=4864, max_sequences=1)
    slot = engine.open()
    got = engine.step([Entry(slot, tokens, [0, 299])])
    assert_close(got, want, "bfloat16", "first positions of the long prompt")

"""The byte and FLOP models behind every roofline fraction, at the real sizes, without a GPU:
the models are bound to tensors on torch's ``meta`` device (shapes and dtypes, no storage)."""
from __future__ import annotations

import pytest
import torch

from thintensor_b200.benchmark import (SHAPES, attention_flops, kv_bytes_per_token, kv_read_bytes_per_token, linear_flops_per_token,
                                       prefill_flops, weight_bytes_per_step)
from thintensor_b200.config.registry import load_config
from thintensor_b200.engine.model import DecoderModel


def meta_model(shape: str) -> DecoderModel:
    arch, config = load_config(SHAPES[shape])
    model = DecoderModel(arch.describe(config), torch.bfloat16, None)
    tensors = {}
    for name, decl in model.weight_declarations().items():
        if decl.alias_of is not None and decl.prefer_alias:
            continue
        tensors[name] = torch.empty(decl.shape, dtype=torch.bfloat16, device="meta")
    model.bind(tensors)
    return model


def test_llama_1b_counts():
    model = meta_model("llama-3.2-1b")
    # 60,817,408 matrix parameters per layer x 16 layers = 973,078,528 multiply-adds per token
    assert linear_flops_per_token(model) == 2 * 973_078_528
    # matrices and head in bfloat16: 2 x (973,078,528 + 262,668,288) bytes; 33 norm weights of 2,048 numbers,
    # which the engine keeps in float32
    matrices = 2 * (973_078_528 + 262_668_288)
    assert weight_bytes_per_step(model) == matrices + 33 * 2048 * 4
    assert abs(weight_bytes_per_step(model) - 2_471.6e6) < 0.2e6
    assert kv_bytes_per_token(model) == 32_768 and kv_read_bytes_per_token(model) == 32_768
    # a 2,048-token prompt: 3.986e12 in the projections, 2.75e11 in causal attention, 5.25e8 in the head
    assert linear_flops_per_token(model) * 2048 == pytest.approx(3.986e12, rel=1e-3)
    assert attention_flops(model, 2048) == pytest.approx(2.75e11, rel=2e-3)
    assert prefill_flops(model, 2048) == pytest.approx(4.261e12, rel=1e-3)


@pytest.mark.parametrize("shape,per_layer,head,kv", [
    ("llama-3.2-3b", 100_663_296, 394_002_432, 114_688),
    ("llama-3.1-8b", 218_103_808, 525_336_576, 131_072),
])
def test_larger_shapes_count_every_matrix_once(shape, per_layer, head, kv):
    model = meta_model(shape)
    layers = len(model.spec.schedule)
    hidden = model.spec.hidden_size
    assert linear_flops_per_token(model) == 2 * per_layer * layers
    assert weight_bytes_per_step(model) == 2 * (per_layer * layers + head) + (2 * layers + 1) * hidden * 4
    assert kv_read_bytes_per_token(model) == kv

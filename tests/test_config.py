"""Configuration and registry: keys, aliases, defaults, errors."""
from __future__ import annotations

import json

import pytest

from conftest import TINY
from thintensor_b200.config import ConfigError, LlamaConfig, load_config, resolve_architecture, supported_architectures


def test_tiny_configurations_differ_everywhere():
    a, b = LlamaConfig.from_dict(TINY["a"]), LlamaConfig.from_dict(TINY["b"])
    for field in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings", "rope_scaling"):
        assert getattr(a, field) != getattr(b, field), field
    assert a.num_attention_heads // a.num_key_value_heads != b.num_attention_heads // b.num_key_value_heads


def test_defaults_follow_the_reference():
    config = LlamaConfig.from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": 128, "num_attention_heads": 4,
                                    "num_hidden_layers": 1, "intermediate_size": 256, "vocab_size": 100})
    assert config.num_key_value_heads == 4          # kv heads default to heads
    assert config.head_dim == 32                    # hidden // heads
    assert config.rms_norm_eps == 1e-6 and config.rope_theta == 10000.0
    assert config.tie_word_embeddings is False and config.rope_scaling is None
    assert config.hidden_act == "silu" and not config.attention_bias and not config.mlp_bias


def test_aliases_and_rope_parameters():
    config = LlamaConfig.from_dict({"model_type": "llama", "n_embd": 64, "n_head": 4, "n_layer": 2, "ffn_dim": 96, "n_vocab": 50,
                                    "num_kv_heads": 2, "rope_parameters": {"type": "llama3", "rope_theta": 5000.0, "factor": 2.0,
                                                                           "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                                                           "original_max_position_embeddings": 32}})
    assert (config.hidden_size, config.num_attention_heads, config.num_hidden_layers, config.intermediate_size, config.vocab_size) == (64, 4, 2, 96, 50)
    assert config.num_key_value_heads == 2 and config.rope_theta == 5000.0
    assert config.rope_scaling.rope_type == "llama3" and config.rope_scaling.original_max_position_embeddings == 32


def test_round_trip_through_config_json(tmp_path):
    for name in TINY:
        config = LlamaConfig.from_dict(TINY[name])
        (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
        arch, again = load_config(tmp_path)
        assert again == config and arch.name == "LlamaForCausalLM"


def test_text_config_of_a_multimodal_wrapper():
    inner = dict(TINY["a"])
    inner.pop("architectures")
    config = LlamaConfig.from_dict({"architectures": ["LlamaForCausalLM"], "text_config": inner, "tie_word_embeddings": False})
    assert config.hidden_size == 64 and config.tie_word_embeddings is False


@pytest.mark.parametrize("change,needle", [
    ({"hidden_size": None}, "missing required field 'hidden_size'"),
    ({"vocab_size": None}, "missing required field 'vocab_size'"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"head_dim": 15}, "must be even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_scaling type 'yarn'"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "missing"),
    ({"num_hidden_layers": 0}, "must be positive"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
])
def test_config_errors(change, needle):
    raw = dict(TINY["a"])
    raw.update(change)
    raw = {k: v for k, v in raw.items() if v is not None}
    with pytest.raises(ConfigError) as err:
        LlamaConfig.from_dict(raw)
    assert needle in str(err.value)


def test_registry():
    assert supported_architectures() == ["LlamaForCausalLM"]
    assert resolve_architecture({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "Tiny-Llama"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError) as err:
        resolve_architecture({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3"})
    assert "Qwen3ForCausalLM" in str(err.value) and "LlamaForCausalLM" in str(err.value)
    with pytest.raises(ConfigError):
        load_config("/nonexistent/folder")


def test_description_is_data():
    """The model description carries every size as a parameter, layer by layer."""
    arch, config = load_config(TINY["b"])
    spec = arch.describe(config)
    assert len(spec.layers) == 3 and [run.layer for run in spec.schedule] == [0, 1, 2]
    mixer = spec.layers[1].parts["mixer"]
    assert mixer.kind == "attention" and mixer.prefix == "model.layers.1.self_attn."
    assert mixer.params["heads"] == 3 and mixer.params["kv_heads"] == 1 and mixer.params["head_dim"] == 32
    assert mixer.params["position"].params["scaling"]["factor"] == 8.0
    assert spec.layers[0].parts["ffn"].params == {"hidden": 96, "inter": 320, "bias": False}
    assert spec.final_norm.params["eps"] == 1e-6 and spec.head.params["tied"] is False


def test_named_shapes_are_whole_configurations():
    """The named benchmark shapes are config.json dicts kept as data; the command line offers
    exactly those names and each of them gives a valid typed configuration."""
    from pathlib import Path

    from thintensor_b200.cli import SHAPE_NAMES

    file = Path(__file__).resolve().parent.parent / "thintensor_b200" / "config" / "shapes.json"
    shapes = json.loads(file.read_text())
    assert tuple(shapes) == SHAPE_NAMES
    for name, raw in shapes.items():
        arch, config = load_config(raw)
        assert arch.name == "LlamaForCausalLM" and config.hidden_size == raw["hidden_size"], name
    one_b = load_config(shapes["llama-3.2-1b"])[1]
    assert (one_b.num_hidden_layers, one_b.num_attention_heads, one_b.num_key_value_heads, one_b.head_dim) == (16, 32, 8, 64)


def test_stop_ids_come_from_both_files(tmp_path):
    """End-of-sequence ids: config.json's (int or list) and generation_config.json's, without
    duplicates; a model that was not read from a folder looks at no file."""
    from thintensor_b200.runtime import stop_ids_of

    config = LlamaConfig.from_dict(dict(TINY["b"]))                      # eos_token_id [3, 11]
    assert stop_ids_of(None, config) == (3, 11)
    assert stop_ids_of(tmp_path, config) == (3, 11)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [11, 17]}))
    assert stop_ids_of(tmp_path, config) == (3, 11, 17)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5}))
    assert stop_ids_of(tmp_path, LlamaConfig.from_dict(dict(TINY["a"]))) == (7, 5)


def test_run_command_takes_random_weights():
    from thintensor_b200.cli import build_parser

    args = build_parser().parse_args(["run", "folder", "--prompt-token-ids", "1,2", "--random-weights", "3", "--steps", "4"])
    assert args.random_weights == 3 and args.max_new_tokens == 4 and args.prompt_token_ids == ["1,2"]
    assert build_parser().parse_args(["run", "folder"]).random_weights is None

"""Weights: safetensors round trip, binding by name, the one error that lists missing,
unexpected and mis-shaped tensors, dtype rules, random model folders."""
from __future__ import annotations

import json

import pytest
import torch

import plain_llama
from conftest import TINY
from thintensor_b200.config import load_config
from thintensor_b200.engine.model import DecoderModel
from thintensor_b200.weights import Checkpoint, WeightError, check, compare, random_tensors, target_dtype, write_model_folder, write_safetensors


def declared_for(name):
    arch, config = load_config(TINY[name])
    return config, DecoderModel(arch.describe(config), torch.float32, None).weight_declarations()


def test_safetensors_round_trip(tmp_path):
    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
        "d": torch.randn(2, 2).to(torch.float16), "scalar": torch.tensor(3.5), "empty": torch.empty(0, 4),
    }
    write_safetensors(tmp_path / "model.safetensors", tensors, metadata={"format": "pt"})
    checkpoint = Checkpoint(tmp_path)
    assert set(checkpoint.entries) == set(tensors)
    for name, tensor in tensors.items():
        got = checkpoint.tensor(name)
        assert got.dtype == tensor.dtype and got.shape == tensor.shape and torch.equal(got, tensor)
    checkpoint.close()
    # the oracle's own reader agrees
    mine = plain_llama.read_safetensors(tmp_path / "model.safetensors")
    assert torch.equal(mine["b"], tensors["b"].double()) and torch.equal(mine["c"], tensors["c"].long())


def test_sharded_checkpoint(tmp_path):
    write_safetensors(tmp_path / "s1.safetensors", {"x": torch.ones(2)})
    write_safetensors(tmp_path / "s2.safetensors", {"y": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    checkpoint = Checkpoint(tmp_path)
    assert torch.equal(checkpoint.tensor("y"), torch.zeros(3)) and set(checkpoint.entries) == {"x", "y"}
    checkpoint.close()
    (tmp_path / "s2.safetensors").unlink()
    with pytest.raises(WeightError, match="s2.safetensors"):
        Checkpoint(tmp_path)


def test_broken_files(tmp_path):
    with pytest.raises(WeightError, match="neither"):
        Checkpoint(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{not json......}")
    with pytest.raises(WeightError, match="not valid JSON"):
        Checkpoint(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"\xff" * 8)
    with pytest.raises(WeightError, match="exceeds"):
        Checkpoint(tmp_path)


def test_declared_names_are_the_checkpoint_names():
    _, declared = declared_for("b")
    assert "model.embed_tokens.weight" in declared and "model.norm.weight" in declared and "lm_head.weight" in declared
    assert declared["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert declared["model.layers.0.mlp.down_proj.weight"].shape == (96, 320)
    assert len(declared) == 3 + 9 * 3


def test_one_error_lists_everything(tmp_path):
    _, declared = declared_for("a")
    tensors = random_tensors(declared, 0, torch.float32)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)      # ignored, not unexpected
    stored = {k: tuple(v.shape) for k, v in tensors.items()}
    missing, unexpected, wrong = compare(declared, stored)
    assert missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert unexpected == ["model.layers.7.extra.weight"]
    assert len(wrong) == 1 and "q_proj" in wrong[0] and "[64, 63]" in wrong[0] and "[64, 64]" in wrong[0]
    with pytest.raises(WeightError) as err:
        check(declared, stored, "somewhere")
    text = str(err.value)
    assert "missing tensors (2)" in text and "unexpected tensors (1)" in text and "wrong shapes (1)" in text
    assert "model.norm.weight" in text and "model.layers.7.extra.weight" in text


def test_tied_and_untied_heads():
    _, tied = declared_for("a")
    stored = {k: d.shape for k, d in tied.items() if k != "lm_head.weight"}
    assert compare(tied, stored) == ([], [], [])
    stored["lm_head.weight"] = tied["lm_head.weight"].shape       # a stored copy of a tied head is ignored
    assert compare(tied, stored) == ([], [], [])
    _, untied = declared_for("b")
    stored = {k: d.shape for k, d in untied.items()}
    assert compare(untied, stored) == ([], [], [])
    del stored["lm_head.weight"]                                   # the reference falls back to the table
    assert compare(untied, stored) == ([], [], [])
    del stored["model.embed_tokens.weight"]
    assert "model.embed_tokens.weight" in compare(untied, stored)[0]


def test_dtype_rule():
    assert target_dtype(torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert target_dtype(torch.float16, torch.bfloat16) == torch.bfloat16
    assert target_dtype(torch.float32, torch.bfloat16) == torch.float32      # stored in 32-bit stays so
    assert target_dtype(torch.bfloat16, torch.float32) == torch.float32
    assert target_dtype(torch.int64, torch.bfloat16) == torch.int32


@pytest.mark.parametrize("name", ["a", "b"])
def test_random_model_folder(tmp_path, name):
    config, declared = declared_for(name)
    folder = write_model_folder(tmp_path / "m", config, declared, seed=3, dtype="bfloat16")
    arch, again = load_config(folder)
    assert again.to_dict() == dict(config.to_dict(), torch_dtype="bfloat16")
    checkpoint = Checkpoint(folder)
    stored = {k: e.shape for k, e in checkpoint.entries.items()}
    check(declared, stored, str(folder))
    assert ("lm_head.weight" in stored) == (not config.tie_word_embeddings)
    assert all(e.dtype == "BF16" for e in checkpoint.entries.values())
    norm = checkpoint.tensor("model.norm.weight").float()
    matrix = checkpoint.tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert abs(float(norm.mean()) - 1.0) < 0.1 and 0.05 < float(norm.std()) < 0.15
    assert abs(float(matrix.mean())) < 0.002 and 0.018 < float(matrix.std()) < 0.022
    checkpoint.close()
    other = write_model_folder(tmp_path / "n", config, declared, seed=3, dtype="bfloat16")
    assert (folder / "model.safetensors").read_bytes() == (other / "model.safetensors").read_bytes()
    third = write_model_folder(tmp_path / "o", config, declared, seed=4, dtype="float32")
    assert (folder / "model.safetensors").read_bytes() != (third / "model.safetensors").read_bytes()
    cfg, weights = plain_llama.read_model(third)
    assert plain_llama.forward(cfg, weights, [1, 2, 3]).shape == (3, config.vocab_size)


def test_wrapper_checkpoints_are_read_without_their_prefix(tmp_path):
    """A multimodal wrapper's folder: the decoder's numbers under ``text_config``, its tensors
    under ``language_model.`` or ``model.language_model.``, other towers beside them.  The decoder
    is found under its plain names, the other towers are left alone, a missing tensor is still named."""
    from thintensor_b200.weights import load_checkpoint
    from thintensor_b200.weights.loader import decoder_names

    config, declared = declared_for("b")
    tensors = random_tensors(declared, 5, torch.float32)
    stored = {}
    for name, tensor in tensors.items():
        if name == "lm_head.weight":
            stored["language_model.lm_head.weight"] = tensor
        elif name.startswith("model.layers.1."):
            stored["model.language_model." + name[len("model."):]] = tensor      # the form without the inner "model."
        else:
            stored["language_model." + name] = tensor
    stored["vision_tower.patch_embedding.weight"] = torch.zeros(4, 4)
    stored["multi_modal_projector.linear.weight"] = torch.zeros(2, 2)
    names = decoder_names(list(stored))
    assert set(names) == set(tensors) and names["model.layers.1.mlp.up_proj.weight"] == "model.language_model.layers.1.mlp.up_proj.weight"
    folder = tmp_path / "wrapper"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps({"model_type": "llama", "text_config": TINY["b"]}))
    write_safetensors(folder / "model.safetensors", stored)
    arch, again = load_config(folder)
    assert again.hidden_size == config.hidden_size
    loaded = load_checkpoint(folder, declared, torch.float32, "cpu", wrapped=True)
    assert set(loaded) == set(tensors) and all(torch.equal(loaded[k], tensors[k]) for k in tensors)
    with pytest.raises(WeightError, match="unexpected tensors"):                 # read as a plain folder nothing fits
        load_checkpoint(folder, declared, torch.float32, "cpu")
    del stored["language_model.model.norm.weight"]
    write_safetensors(folder / "model.safetensors", stored)
    with pytest.raises(WeightError, match=r"missing tensors \(1\): model.norm.weight"):
        load_checkpoint(folder, declared, torch.float32, "cpu", wrapped=True)
    with pytest.raises(WeightError, match="both stand for"):
        decoder_names(["language_model.model.norm.weight", "model.language_model.norm.weight"])

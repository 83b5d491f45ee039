"""The parts' declared interfaces, without a device: what a mixer may ask of the cache, what a
position encoding must say about itself, and how an arrangement with two mixers is given a cache
and states for each."""
from __future__ import annotations

from dataclasses import replace

import pytest
import torch

from conftest import TINY
from thintensor_b200.config.registry import load_config
from thintensor_b200.engine.model import DecoderModel
from thintensor_b200.parts import ARRANGEMENTS, MIXERS, POSITION_ENCODINGS
from thintensor_b200.parts.base import Arrangement, Delta, KVNeed, Mixer, PositionEncoding, StateNeed
from thintensor_b200.parts.spec import LayerSpec, PartSpec, Run


def llama_spec(name):
    arch, config = load_config(TINY[name])
    return arch.describe(config)


def test_attention_refuses_a_position_encoding_it_cannot_apply():
    @POSITION_ENCODINGS.register("toy_learned")
    class Learned(PositionEncoding):
        kind = "learned_table"

        def __init__(self, head_dim):
            self.head_dim = head_dim

    try:
        with pytest.raises(ValueError, match="rotary position encodings or none, not one of kind 'learned_table'"):
            MIXERS.build("attention", {"hidden": 64, "heads": 4, "kv_heads": 2, "head_dim": 16,
                                       "position": PartSpec("toy_learned", {"head_dim": 16})})
        with pytest.raises(NotImplementedError, match="no rotary table"):
            Learned(16).rotary()
    finally:
        POSITION_ENCODINGS.unregister("toy_learned")
    rope = POSITION_ENCODINGS.build("rope", {"head_dim": 16, "theta": 10000.0})
    assert rope.kind == "rotary" and POSITION_ENCODINGS.build("none", {"head_dim": 16}).kind == "none"
    rope.bind({}, torch.float32, None)
    table = rope.rotary()
    assert table.rotary_dim == 16 and table.inv_freq.shape == (8,) and table.attention_scaling == 1.0


def test_a_layer_with_two_mixers_gets_a_cache_and_states_for_each():
    """An arrangement that runs an attention and a recurrent toy mixer side by side: the model asks
    the cache for keys for the one and two states of different dtype for the other, per run, and a
    run that reads another run's cache maps mixer to mixer."""

    @MIXERS.register("toy_recurrent")
    class Recurrent(Mixer):
        def __init__(self, hidden):
            self.hidden = hidden

        def state_needs(self):
            return [StateNeed((self.hidden, 3), torch.bfloat16), StateNeed((2, self.hidden, self.hidden), torch.float32)]

        def forward(self, ctx, x, cache, states):
            return Delta(None)

    @ARRANGEMENTS.register("toy_side_by_side")
    class SideBySide(Arrangement):
        roles = {"norm": "norm", "attention": "mixer", "recurrent": "mixer", "ffn": "ffn"}

        def mixers(self):
            return [self.parts["attention"], self.parts["recurrent"]]

    try:
        spec = llama_spec("a")
        base = spec.layers[0].parts
        layer = LayerSpec("toy_side_by_side", {"norm": base["mixer_norm"], "attention": base["mixer"],
                                               "recurrent": PartSpec("toy_recurrent", {"hidden": 64}), "ffn": base["ffn"]})
        spec = replace(spec, layers=(layer, spec.layers[1]), schedule=(Run(0), Run(1), Run(0, cache_from=0)))
        model = DecoderModel(spec, torch.float32, None)
        kv, states, source = model.cache_needs()
        assert model.users == [[0, 1], [2], [3, 4]]
        assert kv == [KVNeed(2, 16), None, KVNeed(2, 16), KVNeed(2, 16), None]
        assert [len(s) for s in states] == [0, 2, 0, 0, 2] and states[1][0].dtype == torch.bfloat16 and states[1][1].dtype == torch.float32
        assert source == [None, None, None, 0, None]           # keys are shared, states never
        cache = model.new_cache(4, 2, device=None)
        assert [g.runs for g in cache.kv_groups] == [[0, 2]]
        assert sorted(len(g.runs) for g in cache.state_groups) == [2, 2]          # each state shape: one tensor per run that holds it
        assert cache.run_cache(3).group == 0 and not cache.run_cache(3).writes and cache.run_cache(1).group is None
    finally:
        MIXERS.unregister("toy_recurrent")
        ARRANGEMENTS.unregister("toy_side_by_side")

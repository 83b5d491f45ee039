"""Each part alone against the plain implementation's function for it, and the
generality of the assembly: a schedule that names a layer twice and lets a run read
another run's cache, a windowed mixer beside full ones, and a toy mixer with state of
its own that is defined here, registered, built and stepped without touching the
library's files."""
from __future__ import annotations

import pytest
import torch

import plain_llama
from conftest import TINY, token_ids

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make_engine(spec, dtype=torch.float32, seed=0, blocks=16, slots=4, scale=None):
    from thintensor_b200.engine.engine import Engine
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.weights.random_init import random_tensors

    model = DecoderModel(spec, dtype, DEV)
    tensors = random_tensors(model.weight_declarations(), seed, torch.float32)
    for key in tensors:
        if scale and any(key.endswith(s) for s in scale):
            tensors[key] = tensors[key] * scale[[s for s in scale if key.endswith(s)][0]]
    host = {k: v.clone() for k, v in tensors.items()}
    model.bind({k: v.to(DEV).to(dtype if v.is_floating_point() else v.dtype) for k, v in tensors.items()})
    return Engine(model, model.new_cache(blocks, slots)), host


def context_for(engine, slots, news):
    """A StepContext for sequences that bring ``news`` tokens each (cache reserved)."""
    from thintensor_b200.engine.engine import Entry

    entries = [Entry(s, [0] * n, []) for s, n in zip(slots, news)]
    for e in entries:
        engine.cache.reserve(e.slot, engine.cache.length(e.slot) + len(e.tokens))
    ctx, _, _ = engine._prepare(entries, engine.validate(entries), [(i, 0, n) for i, n in enumerate(news)], [0] * len(news))
    return ctx


SHARP = {"q_proj.weight": 8.0, "k_proj.weight": 8.0, "embed_tokens.weight": 20.0, "lm_head.weight": 20.0}


def llama_spec(name):
    from thintensor_b200.config import load_config

    arch, config = load_config(TINY[name])
    return arch.describe(config)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from thintensor_b200.parts import NORMS
    from thintensor_b200.parts.base import Delta

    engine, _ = make_engine(llama_spec("a"), dtype)
    norm = NORMS.build("rmsnorm", {"dim": 200, "eps": 1e-5})
    weight = torch.randn(200) * 0.1 + 1
    norm.bind({"weight": weight.to(DEV)}, dtype, torch.device(DEV))
    ctx = context_for(engine, [engine.open()], [6])
    residual = torch.randn(6, 200, device=DEV)
    delta = torch.randn(2, 6, 200, device=DEV)
    want_residual = residual.double() + delta.double().sum(0)
    out = torch.empty(6, 200, dtype=dtype, device=DEV)
    norm.forward(ctx, residual, Delta(delta), out)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(out.double(), plain_llama.rms_norm(want_residual, weight.double().to(DEV), 1e-5), rtol=tol, atol=tol)
    torch.testing.assert_close(residual.double(), want_residual, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["b", "c"])
def test_attention_and_ffn_parts(name, dtype):
    """The mixer and the feed-forward of layer 0, run alone on packed sequences (one of
    them in two steps), against plain_llama.attention_block and plain_llama.swiglu."""
    spec = llama_spec(name)
    engine, host = make_engine(spec, dtype, seed=3, scale=SHARP)
    cfg = plain_llama.normalise_config(TINY[name])
    weights = {k: (v.to(dtype).double() if v.is_floating_point() else v) for k, v in host.items()}
    inv_freq = plain_llama.rope_inv_freq(cfg["head_dim"], cfg["theta"], cfg["scaling"])
    arrangement = engine.model.layers[0]
    mixer, ffn = arrangement.parts["mixer"], arrangement.parts["ffn"]
    lengths = [70, 3, 130]
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(n, cfg["hidden"], generator=g).to(dtype) for n in lengths]
    slots = [engine.open() for _ in lengths]
    tol = 3e-5 if dtype == torch.float32 else 3e-2

    # step 1: all but the last 2 tokens of sequence 2; step 2: its last 2 tokens alone
    first = [70, 3, 128]
    ctx = context_for(engine, slots, first)
    x = torch.cat([xs[i][: first[i]] for i in range(3)]).to(DEV)
    got = mixer.forward(ctx, x, engine.cache.run_cache(0), []).tensor.sum(0).double().cpu()
    for s, n in zip(slots, first):
        engine.cache.advance(s, n)
    wants = [plain_llama.attention_block(xs[i].double(), weights, "model.layers.0.self_attn.", cfg, torch.arange(lengths[i]), inv_freq)
             for i in range(3)]
    torch.testing.assert_close(got, torch.cat([wants[i][: first[i]] for i in range(3)]), rtol=tol, atol=tol)
    ctx = context_for(engine, [slots[2]], [2])
    got = mixer.forward(ctx, xs[2][128:].to(DEV), engine.cache.run_cache(0), []).tensor.sum(0).double().cpu()
    torch.testing.assert_close(got, wants[2][128:], rtol=tol, atol=tol)

    ctx = context_for(engine, [slots[1]], [5])
    x = torch.randn(5, cfg["hidden"], generator=g).to(dtype)
    got = ffn.forward(ctx, x.to(DEV)).tensor.sum(0).double().cpu()
    torch.testing.assert_close(got, plain_llama.swiglu(x.double(), weights, "model.layers.0.mlp."), rtol=tol, atol=tol)
    engine.check_status()


def test_position_encoding_and_embedding_parts():
    from thintensor_b200.parts import EMBEDDINGS, POSITION_ENCODINGS

    scaling = TINY["c"]["rope_scaling"]
    rope = POSITION_ENCODINGS.build("rope", {"head_dim": 48, "theta": 250000.0, "scaling": scaling})
    torch.testing.assert_close(rope.inv_freq_host, plain_llama.rope_inv_freq(48, 250000.0, scaling), rtol=2e-7, atol=0)
    partial = POSITION_ENCODINGS.build("rope", {"head_dim": 64, "theta": 10000.0, "rotary_dim": 32})
    torch.testing.assert_close(partial.inv_freq_host, plain_llama.rope_inv_freq(32, 10000.0, None))
    with pytest.raises(ValueError):
        POSITION_ENCODINGS.build("rope", {"head_dim": 64, "theta": 10000.0, "rotary_dim": 33})
    engine, _ = make_engine(llama_spec("a"))
    table = torch.randn(50, 24)
    embedding = EMBEDDINGS.build("table", {"vocab": 50, "hidden": 24, "scale": 2.0})
    embedding.bind({"weight": table.to(DEV)}, torch.float32, torch.device(DEV))
    ctx = context_for(engine, [engine.open()], [4])
    tokens = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    residual = torch.empty(4, 24, device=DEV)
    embedding.forward(ctx, tokens, residual)
    torch.testing.assert_close(residual.cpu(), plain_llama.embed(table, [3, 49, 0, 3]) * 2.0)


def plain_schedule(cfg, w, tokens, schedule, windows):
    """The plain implementation's parts run in the order of ``schedule``: entries are
    (layer, cache_from); a run that reads another run's cache attends over that run's
    keys and values with its own queries."""
    positions = torch.arange(len(tokens))
    inv_freq = plain_llama.rope_inv_freq(cfg["head_dim"], cfg["theta"], cfg["scaling"])
    h = plain_llama.embed(w["model.embed_tokens.weight"], tokens)
    kept = {}
    for index, (layer, source) in enumerate(schedule):
        p = f"model.layers.{layer}."
        x = plain_llama.rms_norm(h, w[p + "input_layernorm.weight"], cfg["eps"])
        q, k, v = plain_llama.projections(x, w, p + "self_attn.", cfg, positions, inv_freq)
        if source is not None:
            k, v = kept[source]
        kept[index] = (k, v)
        h = h + plain_llama.output_projection(plain_llama.causal_attention(q, k, v, windows.get(layer)), w, p + "self_attn.")
        h = h + plain_llama.swiglu(plain_llama.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")
    return plain_llama.head(plain_llama.rms_norm(h, w["model.norm.weight"], cfg["eps"]), w)


def test_schedule_repeats_layers_shares_caches_and_mixes_windows():
    """Layer 1 has a window of 40 keys, layers 0 and 2 see everything; the schedule runs
    layer 0 twice and ends with a run of layer 2 that reads the first run's cache.  Whole
    sequences and token-by-token decoding agree with the plain parts run in that order."""
    from dataclasses import replace

    from thintensor_b200.engine.engine import Entry
    from thintensor_b200.parts.spec import PartSpec, Run

    spec = llama_spec("b")
    layers = list(spec.layers)
    mixer = layers[1].parts["mixer"]
    layers[1] = replace(layers[1], parts={**layers[1].parts, "mixer": PartSpec(mixer.kind, {**mixer.params, "window": 40}, mixer.prefix)})
    schedule = (Run(0), Run(1), Run(0), Run(2, cache_from=0))
    spec = replace(spec, layers=tuple(layers), schedule=schedule)
    engine, host = make_engine(spec, torch.float32, seed=7, scale=SHARP, blocks=24)
    assert [g.need.window for g in engine.cache.kv_groups] == [None, 40]
    cfg = plain_llama.normalise_config(TINY["b"])
    weights = {k: v.double() for k, v in host.items()}
    tokens = token_ids(cfg["vocab"], 150, 77)
    want = plain_schedule(cfg, weights, tokens, [(0, None), (1, None), (0, None), (2, 0)], {1: 40})
    slot = engine.open()
    whole = engine.step([Entry(slot, tokens, list(range(len(tokens))))])
    engine.close(slot)
    scale = float(want.abs().max())
    assert float((whole.double().cpu() - want).abs().max()) <= 2e-4 * scale
    slot = engine.open()
    got = [engine.step([Entry(slot, tokens[:100], [99])])]
    for t in range(100, 150):
        got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
    windowed = engine.cache.kv_groups[1].table
    assert windowed.row(slot)[0] == -1 and windowed.pool.held_count < 3      # blocks that slid out of the window went back
    engine.close(slot)
    engine.check_status()
    assert float((torch.cat(got).double().cpu() - want[99:]).abs().max()) <= 2e-4 * scale
    assert engine.cache.free_blocks == engine.cache.num_blocks


def test_toy_mixer_with_state_of_its_own():
    """A mixer that keeps, per sequence, the running sum of its inputs (float32) and their count
    (int32): two fixed-size states of different shape and dtype, no keys.  It outputs
    W @ (mean of the inputs so far).  Defined here, registered here, used for one layer next to
    an attention layer."""
    from dataclasses import replace

    from thintensor_b200.engine.engine import Entry
    from thintensor_b200.parts import MIXERS
    from thintensor_b200.parts.base import Delta, Mixer, StateNeed, WeightDecl
    from thintensor_b200.parts.spec import PartSpec

    @MIXERS.register("toy_running_mean")
    class RunningMean(Mixer):
        def __init__(self, hidden):
            self.hidden = hidden

        def weights(self):
            return {"mix.weight": WeightDecl((self.hidden, self.hidden))}

        def state_needs(self):
            return [StateNeed((self.hidden,), torch.float32), StateNeed((1,), torch.int32)]

        def bind(self, tensors, dtype, device):
            self.w = tensors["mix.weight"].float()

        def forward(self, ctx, x, cache, states):
            total, count = states
            assert total.dtype == torch.float32 and count.dtype == torch.int32 and cache.k_pool is None
            out = torch.empty(1, ctx.n_tokens, self.hidden, dtype=torch.float32, device=x.device)
            at = 0
            for slot, new in zip(ctx.host_slots, ctx.host_new):
                xs = x[at: at + new].float()
                sums = total[slot] + xs.cumsum(0)
                counts = count[slot] + torch.arange(1, new + 1, device=x.device, dtype=torch.int32)
                out[0, at: at + new] = (sums / counts[:, None].float()) @ self.w.T
                total[slot] = sums[-1]
                count[slot] = counts[-1]
                at += new
            return Delta(out)

    try:
        spec = llama_spec("a")
        layers = list(spec.layers)
        layers[0] = replace(layers[0], parts={**layers[0].parts, "mixer": PartSpec("toy_running_mean", {"hidden": 64}, "model.layers.0.toy.")})
        spec = replace(spec, layers=tuple(layers))
        engine, host = make_engine(spec, torch.float32, seed=9, scale=SHARP)
        assert "model.layers.0.toy.mix.weight" in host and "model.layers.0.self_attn.q_proj.weight" not in host
        assert len(engine.cache.state_groups) == 2 and len(engine.cache.kv_groups) == 1
        cfg = plain_llama.normalise_config(TINY["a"])
        w = {k: v.double() for k, v in host.items()}

        def plain(tokens):
            positions = torch.arange(len(tokens))
            inv_freq = plain_llama.rope_inv_freq(cfg["head_dim"], cfg["theta"], cfg["scaling"])
            h = plain_llama.embed(w["model.embed_tokens.weight"], tokens)
            x = plain_llama.rms_norm(h, w["model.layers.0.input_layernorm.weight"], cfg["eps"])
            mean = x.cumsum(0) / torch.arange(1, len(tokens) + 1)[:, None]
            h = h + mean @ w["model.layers.0.toy.mix.weight"].T
            h = h + plain_llama.swiglu(plain_llama.rms_norm(h, w["model.layers.0.post_attention_layernorm.weight"], cfg["eps"]), w, "model.layers.0.mlp.")
            h = plain_llama.decoder_layer(h, w, 1, cfg, positions, inv_freq)
            return plain_llama.head(plain_llama.rms_norm(h, w["model.norm.weight"], cfg["eps"]), w)

        prompts = [token_ids(256, n, 90 + n) for n in (30, 7, 75)]
        wants = [plain(p) for p in prompts]
        slots = [engine.open() for _ in prompts]
        heads = [20, 7, 10]
        logits = engine.step([Entry(s, p[:h], [h - 1]) for s, p, h in zip(slots, prompts, heads)])
        for i in range(3):
            assert float((logits[i].double().cpu() - wants[i][heads[i] - 1]).abs().max()) <= 2e-4 * float(wants[i].abs().max())
        engine.close(slots[1])
        for t in range(10):                       # sequences 0 and 2 go on one token at a time
            logits = engine.step([Entry(slots[0], [prompts[0][20 + t]], [0]), Entry(slots[2], [prompts[2][10 + t]], [0])])
            for row, (i, place) in enumerate([(0, 20 + t), (2, 10 + t)]):
                assert float((logits[row].double().cpu() - wants[i][place]).abs().max()) <= 2e-4 * float(wants[i].abs().max())
        engine.close(slots[0])
        engine.close(slots[2])
        # a slot that is used again starts from zero state
        slot = engine.open()
        logits = engine.step([Entry(slot, prompts[1], [6])])
        assert float((logits[0].double().cpu() - wants[1][6]).abs().max()) <= 2e-4 * float(wants[1].abs().max())
        engine.close(slot)
    finally:
        MIXERS.unregister("toy_running_mean")


def test_toy_feed_forward_with_routing():
    """A feed-forward that routes every token to one of three experts (router logits in
    float32, the expert with the largest logit), defined and registered here and used for
    layer 1 while layer 0 keeps the dense SwiGLU: the loader finds its tensors by name, the
    engine steps it in batches of unequal length, and padding-free packing means a token's
    expert does not depend on its neighbours."""
    from dataclasses import replace

    from thintensor_b200.engine.engine import Entry
    from thintensor_b200.parts import FEED_FORWARDS
    from thintensor_b200.parts.base import Delta, FeedForward, WeightDecl
    from thintensor_b200.parts.spec import PartSpec

    experts, hidden, inter = 3, 64, 40

    @FEED_FORWARDS.register("toy_routed")
    class Routed(FeedForward):
        def __init__(self, hidden, inter, experts):
            self.hidden, self.inter, self.experts = hidden, inter, experts

        def weights(self):
            out = {"router.weight": WeightDecl((self.experts, self.hidden))}
            for e in range(self.experts):
                out[f"experts.{e}.up.weight"] = WeightDecl((self.inter, self.hidden))
                out[f"experts.{e}.down.weight"] = WeightDecl((self.hidden, self.inter))
            return out

        def bind(self, tensors, dtype, device):
            self.router = tensors["router.weight"].float()
            self.up = torch.stack([tensors[f"experts.{e}.up.weight"].float() for e in range(self.experts)])
            self.down = torch.stack([tensors[f"experts.{e}.down.weight"].float() for e in range(self.experts)])

        def forward(self, ctx, x):
            xf = x.float()
            choice = (xf @ self.router.T).argmax(dim=-1)
            hidden_act = torch.relu(torch.einsum("tih,th->ti", self.up[choice], xf))
            return Delta(torch.einsum("thi,ti->th", self.down[choice], hidden_act).unsqueeze(0).contiguous())

    try:
        spec = llama_spec("a")
        layers = list(spec.layers)
        layers[1] = replace(layers[1], parts={**layers[1].parts, "ffn": PartSpec("toy_routed", {"hidden": hidden, "inter": inter, "experts": experts}, "model.layers.1.moe.")})
        spec = replace(spec, layers=tuple(layers))
        engine, host = make_engine(spec, torch.float32, seed=13, scale={**SHARP, "router.weight": 30.0})
        assert "model.layers.1.moe.experts.2.down.weight" in host and "model.layers.1.mlp.gate_proj.weight" not in host
        cfg = plain_llama.normalise_config(TINY["a"])
        w = {k: v.double() for k, v in host.items()}

        def plain(tokens):
            positions = torch.arange(len(tokens))
            inv_freq = plain_llama.rope_inv_freq(cfg["head_dim"], cfg["theta"], cfg["scaling"])
            h = plain_llama.embed(w["model.embed_tokens.weight"], tokens)
            h = plain_llama.decoder_layer(h, w, 0, cfg, positions, inv_freq)
            p = "model.layers.1."
            h = h + plain_llama.attention_block(plain_llama.rms_norm(h, w[p + "input_layernorm.weight"], cfg["eps"]), w, p + "self_attn.", cfg, positions, inv_freq)
            x = plain_llama.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"])
            choice = (x @ w[p + "moe.router.weight"].T).argmax(dim=-1)
            rows = []
            for t in range(len(tokens)):
                e = int(choice[t])
                rows.append(w[p + f"moe.experts.{e}.down.weight"] @ torch.relu(w[p + f"moe.experts.{e}.up.weight"] @ x[t]))
            h = h + torch.stack(rows)
            return plain_llama.head(plain_llama.rms_norm(h, w["model.norm.weight"], cfg["eps"]), w), choice

        prompts = [token_ids(256, n, 130 + n) for n in (40, 3, 66)]
        assert len({int(c) for p in prompts for c in plain(p)[1]}) == experts, "the prompts should reach every expert"
        slots = [engine.open() for _ in prompts]
        heads = [30, 3, 50]
        logits = engine.step([Entry(s, p[:h], list(range(h))) for s, p, h in zip(slots, prompts, heads)])
        at = 0
        for i, h in enumerate(heads):
            want = plain(prompts[i])[0]
            assert float((logits[at: at + h].double().cpu() - want[:h]).abs().max()) <= 2e-4 * float(want.abs().max())
            at += h
        for t in range(10):
            logits = engine.step([Entry(slots[0], [prompts[0][30 + t]], [0]), Entry(slots[2], [prompts[2][50 + t]], [0])])
            for row, (i, place) in enumerate([(0, 30 + t), (2, 50 + t)]):
                want = plain(prompts[i])[0]
                assert float((logits[row].double().cpu() - want[place]).abs().max()) <= 2e-4 * float(want.abs().max())
        for s in slots:
            engine.close(s)
    finally:
        FEED_FORWARDS.unregister("toy_routed")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_position_encoding(dtype):
    """Another position encoding, defined and registered here: positions divided by a factor
    (linear interpolation) with a rotary part of half the head.  Attention takes it through
    its `position` parameter; nothing in the library changes."""
    from dataclasses import replace

    from thintensor_b200.engine.engine import Entry
    from thintensor_b200.parts import POSITION_ENCODINGS
    from thintensor_b200.parts.base import PositionEncoding, RotaryTable
    from thintensor_b200.parts.spec import PartSpec

    @POSITION_ENCODINGS.register("toy_interpolated")
    class Interpolated(PositionEncoding):
        kind = "rotary"

        def __init__(self, head_dim, theta, factor):
            self.rotary_dim = head_dim // 2
            index = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
            self.table = theta ** (-index / self.rotary_dim) / factor

        def bind(self, tensors, dtype, device):
            self.device_table = self.table.to(device)

        def rotary(self):
            return RotaryTable(self.device_table, self.rotary_dim, 1.0)

    try:
        name = "d"
        spec = llama_spec(name)
        layers = []
        for layer in spec.layers:
            mixer = layer.parts["mixer"]
            position = PartSpec("toy_interpolated", {"head_dim": 64, "theta": 1000.0, "factor": 4.0})
            layers.append(replace(layer, parts={**layer.parts, "mixer": PartSpec(mixer.kind, {**mixer.params, "position": position}, mixer.prefix)}))
        spec = replace(spec, layers=tuple(layers))
        engine, host = make_engine(spec, dtype, seed=17, scale=SHARP)
        cfg = plain_llama.normalise_config(TINY[name])
        w = {k: (v.to(dtype).double() if v.is_floating_point() else v) for k, v in host.items()}
        inv_freq = (1000.0 ** (-torch.arange(0, 32, 2, dtype=torch.float32) / 32) / 4.0)

        def plain(tokens):
            T = len(tokens)
            positions = torch.arange(T)
            cos, sin = plain_llama.rope_cos_sin(inv_freq, positions, torch.float64)
            h = plain_llama.embed(w["model.embed_tokens.weight"], tokens)
            for layer in range(cfg["layers"]):
                p = f"model.layers.{layer}."
                x = plain_llama.rms_norm(h, w[p + "input_layernorm.weight"], cfg["eps"])
                q = (x @ w[p + "self_attn.q_proj.weight"].T).reshape(T, cfg["heads"], 64)
                k = (x @ w[p + "self_attn.k_proj.weight"].T).reshape(T, cfg["kv_heads"], 64)
                v = (x @ w[p + "self_attn.v_proj.weight"].T).reshape(T, cfg["kv_heads"], 64)
                q = torch.cat((plain_llama.apply_rope(q[..., :32], cos, sin), q[..., 32:]), dim=-1)
                k = torch.cat((plain_llama.apply_rope(k[..., :32], cos, sin), k[..., 32:]), dim=-1)
                h = h + plain_llama.output_projection(plain_llama.causal_attention(q, k, v), w, p + "self_attn.")
                h = h + plain_llama.swiglu(plain_llama.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")
            return plain_llama.head(plain_llama.rms_norm(h, w["model.norm.weight"], cfg["eps"]), w)

        tokens = token_ids(cfg["vocab"], 150, 171)
        want = plain(tokens)
        slot = engine.open()
        got = [engine.step([Entry(slot, tokens[:140], list(range(140)))])]
        for t in range(140, 150):
            got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
        engine.close(slot)
        engine.check_status()
        from conftest import assert_close
        assert_close(torch.cat(got), want, "float32" if dtype == torch.float32 else "bfloat16", "toy position encoding")
    finally:
        POSITION_ENCODINGS.unregister("toy_interpolated")


def test_toy_arrangement_with_two_mixers_side_by_side():
    """A layer whose arrangement, defined and registered here, runs an attention and a recurrent toy mixer on the same
    normed input and adds both outputs: the model gives each mixer a cache and states of its own (keys for the one,
    a float32 sum and an int32 count for the other), per run of the schedule; whole prompts in a batch and token by
    token agree with the plain parts wired the same way."""
    from dataclasses import replace

    from thintensor_b200.engine.engine import Entry
    from thintensor_b200.parts import ARRANGEMENTS, MIXERS
    from thintensor_b200.parts.base import Arrangement, Delta, Mixer, StateNeed, WeightDecl
    from thintensor_b200.parts.spec import LayerSpec, PartSpec

    @MIXERS.register("toy_memory")
    class Memory(Mixer):
        def __init__(self, hidden):
            self.hidden = hidden

        def weights(self):
            return {"mix.weight": WeightDecl((self.hidden, self.hidden))}

        def state_needs(self):
            return [StateNeed((self.hidden,), torch.float32), StateNeed((1,), torch.int32)]

        def bind(self, tensors, dtype, device):
            self.w = tensors["mix.weight"].float()

        def forward(self, ctx, x, cache, states):
            total, count = states
            assert cache.k_pool is None, "this mixer asked for no keys"
            out = torch.empty(1, ctx.n_tokens, self.hidden, dtype=torch.float32, device=x.device)
            at = 0
            for slot, new in zip(ctx.host_slots, ctx.host_new):
                sums = total[slot] + x[at: at + new].float().cumsum(0)
                counts = count[slot] + torch.arange(1, new + 1, device=x.device, dtype=torch.int32)
                out[0, at: at + new] = (sums / counts[:, None].float()) @ self.w.T
                total[slot], count[slot] = sums[-1], counts[-1]
                at += new
            return Delta(out)

    @ARRANGEMENTS.register("toy_side_by_side")
    class SideBySide(Arrangement):
        roles = {"norm": "norm", "attention": "mixer", "memory": "mixer", "ffn_norm": "norm", "ffn": "ffn"}

        def mixers(self):
            return [self.parts["attention"], self.parts["memory"]]

        def run(self, ctx, residual, pending, caches, states):
            hidden = residual.shape[-1]
            normed = ctx.scratch("toy.normed", (ctx.n_tokens, hidden))
            self.parts["norm"].forward(ctx, residual, pending, normed)
            a = self.parts["attention"].forward(ctx, normed, caches[0], states[0])
            b = self.parts["memory"].forward(ctx, normed, caches[1], states[1])
            both = Delta(torch.cat([a.tensor, b.tensor]))             # the next norm adds every plane
            self.parts["ffn_norm"].forward(ctx, residual, both, normed)
            return self.parts["ffn"].forward(ctx, normed)

    try:
        spec = llama_spec("a")
        base = spec.layers[0].parts
        layer = LayerSpec("toy_side_by_side", {"norm": base["mixer_norm"], "attention": base["mixer"], "ffn_norm": base["ffn_norm"], "ffn": base["ffn"],
                                               "memory": PartSpec("toy_memory", {"hidden": 64}, "model.layers.0.memory.")})
        spec = replace(spec, layers=(layer, spec.layers[1]))
        engine, host = make_engine(spec, torch.float32, seed=21, scale=SHARP)
        assert not engine.use_step_graphs, "a part that computes on the host keeps the engine from replaying steps"
        assert engine.model.users == [[0, 1], [2]] and len(engine.cache.kv_groups) == 1 and len(engine.cache.state_groups) == 2
        cfg = plain_llama.normalise_config(TINY["a"])
        w = {k: v.double() for k, v in host.items()}

        def plain(tokens):
            positions = torch.arange(len(tokens))
            inv_freq = plain_llama.rope_inv_freq(cfg["head_dim"], cfg["theta"], cfg["scaling"])
            h = plain_llama.embed(w["model.embed_tokens.weight"], tokens)
            p = "model.layers.0."
            x = plain_llama.rms_norm(h, w[p + "input_layernorm.weight"], cfg["eps"])
            mean = x.cumsum(0) / torch.arange(1, len(tokens) + 1)[:, None]
            h = h + plain_llama.attention_block(x, w, p + "self_attn.", cfg, positions, inv_freq) + mean @ w[p + "memory.mix.weight"].T
            h = h + plain_llama.swiglu(plain_llama.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")
            h = plain_llama.decoder_layer(h, w, 1, cfg, positions, inv_freq)
            return plain_llama.head(plain_llama.rms_norm(h, w["model.norm.weight"], cfg["eps"]), w)

        prompts = [token_ids(256, n, 230 + n) for n in (44, 9, 80)]
        wants = [plain(p) for p in prompts]
        slots = [engine.open() for _ in prompts]
        heads = [30, 9, 70]
        logits = engine.step([Entry(s, p[:h], [0, h - 1]) for s, p, h in zip(slots, prompts, heads)])
        for i in range(3):
            got = logits[2 * i: 2 * i + 2].double().cpu()
            assert float((got - wants[i][[0, heads[i] - 1]]).abs().max()) <= 2e-4 * float(wants[i].abs().max())
        engine.close(slots[1])
        for t in range(10):
            logits = engine.step([Entry(slots[0], [prompts[0][30 + t]], [0]), Entry(slots[2], [prompts[2][70 + t]], [0])])
            for row, (i, place) in enumerate([(0, 30 + t), (2, 70 + t)]):
                assert float((logits[row].double().cpu() - wants[i][place]).abs().max()) <= 2e-4 * float(wants[i].abs().max())
        engine.close(slots[0])
        engine.close(slots[2])
        assert engine.cache.free_blocks == engine.cache.num_blocks
    finally:
        MIXERS.unregister("toy_memory")
        ARRANGEMENTS.unregister("toy_side_by_side")

"""Plain, slow implementation of the Llama dense decoder, used only as the test oracle.

Whole sequences, no cache, one function per part, no batching tricks.  It shares no
code with the package under test: it has its own reading of config.json, its own
safetensors reader, its own rotary tables, attention, feed-forward, sampling and
generation.  Every function cites the place in random-unknown-username/Thintensor whose
formula it restates (paths are relative to that project).

Precision.  The reference computes norm statistics, softmax and rotary angles in
float32 and the rest in the model dtype.  The oracle computes everything in ``dtype``
(float64 by default) except the two places where float32 rounding is part of the
*definition* of the function: ``inv_freq`` and the angle ``inv_freq * position`` are
float32 products exactly as in thinruntime/gpu_runtime.py:8736-8772, because an
angle rounded in float32 at a far position differs from the float64 one by more
than the tolerance the tests use.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# --------------------------------------------------------------------------------------
# configuration (thinruntime/model_arch.py:112-295: keys, aliases, defaults)
# --------------------------------------------------------------------------------------


def read_config(folder) -> dict:
    """config.json -> the numbers the model needs, with the reference's defaults.

    thinruntime/model_arch.py:132-142 (kv heads default to heads, head_dim to
    hidden // heads), :158-174 (tie_word_embeddings false, rope_theta 10000,
    rms_norm_eps 1e-6 when absent), :169 (rope_scaling or rope_parameters).
    """
    raw = json.loads((Path(folder) / "config.json").read_text())
    return normalise_config(raw)


def normalise_config(raw: dict) -> dict:
    heads = int(raw["num_attention_heads"])
    hidden = int(raw["hidden_size"])
    scaling = raw.get("rope_scaling") or raw.get("rope_parameters")
    theta = raw.get("rope_theta") or (raw.get("rope_parameters") or {}).get("rope_theta") or 10000.0
    return {
        "vocab": int(raw["vocab_size"]),
        "hidden": hidden,
        "inter": int(raw["intermediate_size"]),
        "layers": int(raw["num_hidden_layers"]),
        "heads": heads,
        "kv_heads": int(raw.get("num_key_value_heads") or heads),
        "head_dim": int(raw.get("head_dim") or hidden // heads),
        "eps": float(raw.get("rms_norm_eps") or 1e-6),
        "theta": float(theta),
        "scaling": scaling,
        "tied": bool(raw.get("tie_word_embeddings", False)),
    }


# --------------------------------------------------------------------------------------
# weights: a minimal safetensors reader of its own
# --------------------------------------------------------------------------------------

_NP_DTYPES = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """name -> float64/int64 tensor.  BF16 is widened by placing its 16 bits in the
    top half of a float32 word (exact)."""
    data = Path(path).read_bytes()
    (header_len,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8 : 8 + header_len].decode("utf-8"))
    base = 8 + header_len
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        begin, end = meta["data_offsets"]
        raw = data[base + begin : base + end]
        shape = tuple(meta["shape"])
        if meta["dtype"] == "BF16":
            half = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            array = half.view(np.float32).astype(np.float64)
        else:
            array = np.frombuffer(raw, dtype=_NP_DTYPES[meta["dtype"]])
            array = array.astype(np.int64 if meta["dtype"].startswith("I") else np.float64)
        out[name] = torch.from_numpy(array.reshape(shape).copy())
    return out


def read_model(folder):
    """(config, weights) of a model folder holding config.json and model.safetensors."""
    return read_config(folder), read_safetensors(Path(folder) / "model.safetensors")


# --------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------


def embed(table: torch.Tensor, tokens) -> torch.Tensor:
    """h0 = E[token], no scaling for Llama (thinruntime/gpu_runtime.py:10072;
    embedding_scale 1.0 at thinruntime/model_arch.py:234-238)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis
    (thinruntime/gpu_runtime.py:13028-13039, weight_offset 0 for Llama)."""
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """float32 inverse frequencies, [head_dim / 2].

    Default: theta ** (-(2i) / head_dim) (thinruntime/gpu_runtime.py:8759-8772).
    llama3: the reference hands the parameters to a library
    (thinruntime/gpu_runtime.py:8779-8816); the rule restated here is the published
    Llama 3.1 one: with wavelength 2*pi/f and L = original_max_position_embeddings,
    wavelengths shorter than L/high_freq_factor keep f, longer than L/low_freq_factor
    use f/factor, and those between are blended linearly in L/wavelength.
    """
    index = torch.arange(0, head_dim, 2, dtype=torch.float32)
    inv_freq = theta ** (-index / head_dim)
    kind = None
    if scaling:
        kind = scaling.get("rope_type") or scaling.get("type")
    if kind in (None, "default"):
        return inv_freq
    if kind != "llama3":
        raise ValueError(f"oracle knows no rope_type {kind!r}")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    out = []
    for f in inv_freq.tolist():
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            t = (original / wavelength - low) / (high - low)
            out.append((1.0 - t) * f / factor + t * f)
    return torch.tensor(out, dtype=torch.float32)


def rope_cos_sin(inv_freq: torch.Tensor, positions: torch.Tensor, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """cos, sin of inv_freq * position, [T, head_dim / 2]; the product is float32
    (thinruntime/gpu_runtime.py:8743-8750, attention scaling 1 for default and llama3)."""
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    angle = angle.to(torch.float64)
    return angle.cos().to(dtype), angle.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, head_dim].  Halves a = x[..., :d/2], b = x[..., d/2:];
    a' = a cos - b sin, b' = b cos + a sin (thinruntime/gpu_runtime.py:8703-8712)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((a * c - b * s, b * c + a * s), dim=-1)


def causal_attention(q, k, v, window: int | None = None) -> torch.Tensor:
    """q: [T, heads, d], k, v: [T, kv_heads, d] of ONE sequence -> [T, heads * d].

    Query head h reads KV head h // (heads / kv_heads); scores scaled by d ** -0.5;
    position t sees keys 0..t (the cache holds exactly those at step t), softmax over
    them, then the weighted sum of values (thinruntime/gpu_runtime.py:8913-8961).
    ``window`` keeps only the last ``window`` keys
    (thinruntime/gpu_runtime.py:4666-4697), unused by Llama.
    """
    T, heads, d = q.shape
    kv_heads = k.shape[1]
    group = heads // kv_heads
    out = torch.zeros(T, heads, d, dtype=q.dtype)
    for h in range(heads):
        kh = h // group
        scores = (q[:, h, :] @ k[:, kh, :].T) * (d ** -0.5)
        t_idx = torch.arange(T)
        hidden = t_idx[None, :] > t_idx[:, None]
        if window is not None:
            hidden = hidden | (t_idx[None, :] <= t_idx[:, None] - window)
        scores = scores.masked_fill(hidden, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ v[:, kh, :]
    return out.reshape(T, heads * d)


def projections(x, w: dict, prefix: str, cfg: dict, positions, inv_freq):
    """q, k, v of one sequence after the rotary encoding: [T, heads, d], [T, kv_heads, d]
    twice (thinruntime/gpu_runtime.py:10151-10209).  Weights are [out_features,
    in_features] applied as W @ x, with optional biases (:10179-10188)."""
    T = x.shape[0]
    heads, kv_heads, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]

    def proj(name):
        y = x @ w[prefix + name + ".weight"].T
        bias = w.get(prefix + name + ".bias")
        return y if bias is None else y + bias

    q = proj("q_proj").reshape(T, heads, d)
    k = proj("k_proj").reshape(T, kv_heads, d)
    v = proj("v_proj").reshape(T, kv_heads, d)
    cos, sin = rope_cos_sin(inv_freq, positions, x.dtype)
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin), v


def output_projection(mixed, w: dict, prefix: str) -> torch.Tensor:
    """a = Wo @ o (+ bias) (thinruntime/gpu_runtime.py:10221-10231)."""
    y = mixed @ w[prefix + "o_proj.weight"].T
    bias = w.get(prefix + "o_proj.bias")
    return y if bias is None else y + bias


def attention_block(x, w: dict, prefix: str, cfg: dict, positions, inv_freq, window=None) -> torch.Tensor:
    """Projections, rotary on q and k, causal attention, output projection
    (thinruntime/gpu_runtime.py:10151-10249)."""
    q, k, v = projections(x, w, prefix, cfg, positions, inv_freq)
    return output_projection(causal_attention(q, k, v, window), w, prefix)


def swiglu(x, w: dict, prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(g) = g / (1 + exp(-g))
    (thinruntime/gpu_runtime.py:10286-10366, activation at :10351), each projection with its
    bias where the checkpoint stores one (:10312-10319 gate and up, :10361-10366 down)."""
    def proj(name, y):
        out = y @ w[prefix + name + ".weight"].T
        bias = w.get(prefix + name + ".bias")
        return out if bias is None else out + bias

    gate, up = proj("gate_proj", x), proj("up_proj", x)
    act = gate / (1.0 + torch.exp(-gate)) * up
    return proj("down_proj", act)


def decoder_layer(h, w: dict, layer: int, cfg: dict, positions, inv_freq) -> torch.Tensor:
    """h += attn(norm(h)); h += mlp(norm(h)) (thinruntime/gpu_runtime.py:10114-10390)."""
    p = f"model.layers.{layer}."
    h = h + attention_block(rms_norm(h, w[p + "input_layernorm.weight"], cfg["eps"]), w, p + "self_attn.", cfg, positions, inv_freq)
    h = h + swiglu(rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")
    return h


def head(h, w: dict) -> torch.Tensor:
    """logits = W_head @ norm(h); the head is lm_head.weight when that tensor exists,
    else the embedding table (thinruntime/gpu_runtime.py:10392-10401)."""
    table = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return h @ table.T


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64) -> torch.Tensor:
    """Logits [T, vocab] of ONE whole sequence, every position, nothing cached."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    positions = torch.arange(len(tokens))
    inv_freq = rope_inv_freq(cfg["head_dim"], cfg["theta"], cfg["scaling"])
    h = embed(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["layers"]):
        h = decoder_layer(h, w, layer, cfg, positions, inv_freq)
    return head(rms_norm(h, w["model.norm.weight"], cfg["eps"]), w)


# --------------------------------------------------------------------------------------
# sampling and generation
# --------------------------------------------------------------------------------------

_MASK64 = (1 << 64) - 1


def _mix64(x: int) -> int:
    """splitmix64 finaliser on a Python integer."""
    x &= _MASK64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _MASK64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _MASK64
    x ^= x >> 31
    return x


def uniform(seed: int, request: int, step: int) -> float:
    """The uniform number in [0, 1) that request ``request`` draws at decode step
    ``step``: three rounds of the splitmix64 finaliser over (seed, request, step),
    top 24 bits.  A function of its three arguments only, so a request's draws do not
    depend on the batch it runs in.  (The reference seeds a host generator with
    seed + step per token, scripts/stress_validate_thin.py:835-837; the counter form
    is this library's own.)"""
    x = _mix64((seed & _MASK64) + 0x9E3779B97F4A7C15)
    x = _mix64(x ^ ((request & _MASK64) * 0xD1B54A32D192ED03 & _MASK64))
    x = _mix64(x ^ ((step & _MASK64) * 0x8CB92BA72F3D8DD7 & _MASK64))
    return (x >> 40) / float(1 << 24)


def sampling_probabilities(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """scores = logits / T; below the k-th largest -> -inf; then the nucleus: sorted
    descending, a token goes when the cumulative probability BEFORE it already
    exceeds top_p; softmax of what is left (scripts/stress_validate_thin.py:840-856)."""
    scores = logits.to(torch.float64) / temperature
    if 0 < top_k < scores.numel():
        threshold = torch.topk(scores, top_k).values[-1]
        scores = scores.masked_fill(scores < threshold, float("-inf"))
    if top_p < 1.0:
        sorted_scores, order = torch.sort(scores, descending=True)
        cumulative = torch.cumsum(torch.softmax(sorted_scores, dim=-1), dim=-1)
        remove = cumulative > top_p
        remove[1:] = remove[:-1].clone()
        remove[0] = False
        scores = scores.clone()
        scores[order[remove]] = float("-inf")
    return torch.softmax(scores, dim=-1)


def select_token(logits, temperature, top_k, top_p, seed, request, step) -> int:
    """Greedy: argmax, lowest id on ties (scripts/stress_validate_thin.py:831-833;
    thinruntime/triton_kernels.py:2249-2250).  Otherwise the inverse CDF of the
    sampling distribution, in token-id order, at uniform(seed, request, step)."""
    if temperature <= 0:
        best = logits.max()
        return int(torch.nonzero(logits == best)[0])
    p = sampling_probabilities(logits, temperature, top_k, top_p)
    cdf = torch.cumsum(p, dim=-1)
    u = uniform(seed, request, step) * float(cdf[-1])
    return min(int(torch.searchsorted(cdf, torch.tensor(u, dtype=cdf.dtype), right=True)), p.numel() - 1)


def generate(cfg, weights, prompt, max_new_tokens, stop_ids=(), temperature=0.0, top_k=0, top_p=1.0,
             seed=0, request=0, dtype=torch.float64) -> list[int]:
    """Recompute the whole sequence for every new token; the stop token is kept in
    the output and ends the sequence (thinruntime/cli.py:2826-2858)."""
    tokens = list(prompt)
    produced = []
    for step in range(max_new_tokens):
        logits = forward(cfg, weights, tokens, dtype)[-1]
        token = select_token(logits, temperature, top_k, top_p, seed, request, step)
        produced.append(token)
        tokens.append(token)
        if token in stop_ids:
            break
    return produced

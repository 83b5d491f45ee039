"""Causal grouped-query attention over the block cache.

For each token: q, k, v projections of the normed hidden state (one fused matrix),
position encoding on q and k, k and v appended to the sequence's cache, softmax
attention of q over every cached key of its sequence (or the last ``window`` of them)
with query head h reading key/value head ``h // (heads / kv_heads)`` and scores scaled
by ``head_dim ** -0.5``, then the output projection
(thinruntime/gpu_runtime.py:10151-10249 and 8913-8961).
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import MIXERS, POSITION_ENCODINGS, Delta, KVNeed, Mixer, RotaryTable, WeightDecl
from .linear import Linear
from .spec import PartSpec


def kv_splits(ctx, parallel_units: int, keys_per_slice: int, target_units: int) -> int:
    """Into how many slices the keys of a decode step are cut so that the grid fills the
    GPU: ``parallel_units`` is how many independent units (warps or CTAs) the step has
    without slicing, ``target_units`` how many the GPU wants.  Depends only on the step's
    shape and the length bound, never on the lengths on the device."""
    if not ctx.decode:
        return 1
    want = target_units // max(parallel_units, 1)
    most = ctx.max_total // keys_per_slice
    return max(1, min(want, most, 64))


@MIXERS.register("attention")
class CausalAttention(Mixer):
    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, position: PartSpec | None = None,
                 bias: bool = False, window: int | None = None, scale: float | None = None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} key/value heads")
        api.check_head_dim(self.head_dim)
        self.bias = bool(bias)
        self.window = None if not window else int(window)
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        position = position or PartSpec("none", {"head_dim": self.head_dim})
        self.position = POSITION_ENCODINGS.build(position.kind, dict(position.params))
        if self.position.kind not in ("rotary", "none"):
            raise ValueError(f"attention applies rotary position encodings or none, not one of kind {self.position.kind!r}")
        self.rot: RotaryTable | None = None         # what the kernels rotate by; rotary_dim 0 switches rotation off
        self.qkv: Linear | None = None
        self.q_only: Linear | None = None
        self.out: Linear | None = None

    # -------------------------------------------------------------- declarations
    def weights(self) -> dict[str, WeightDecl]:
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        out = {
            "q_proj.weight": WeightDecl((q, self.hidden)),
            "k_proj.weight": WeightDecl((kv, self.hidden)),
            "v_proj.weight": WeightDecl((kv, self.hidden)),
            "o_proj.weight": WeightDecl((self.hidden, q)),
        }
        if self.bias:
            out.update({
                "q_proj.bias": WeightDecl((q,)), "k_proj.bias": WeightDecl((kv,)), "v_proj.bias": WeightDecl((kv,)),
                "o_proj.bias": WeightDecl((self.hidden,)),
            })
        return out

    def cache_need(self) -> KVNeed:
        return KVNeed(self.kv_heads, self.head_dim, self.window)

    def bind(self, tensors, dtype, device) -> None:
        self.position.bind({}, dtype, device)
        if self.position.kind == "rotary":
            self.rot = self.position.rotary()
            if self.rot.rotary_dim % 2 or not 0 <= self.rot.rotary_dim <= self.head_dim:
                raise ValueError(f"the rotary part must be even and at most the head size {self.head_dim}, got {self.rot.rotary_dim}")
        else:
            self.rot = RotaryTable(torch.zeros(1, dtype=torch.float32, device=device), 0, 1.0)
        weight = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0)
        bias = None
        if self.bias:
            bias = torch.cat([tensors["q_proj.bias"].float(), tensors["k_proj.bias"].float(), tensors["v_proj.bias"].float()])
        self.qkv = Linear(weight, bias)
        self.q_only = self.qkv.rows(0, self.heads * self.head_dim)
        self.out = Linear(tensors["o_proj.weight"], tensors["o_proj.bias"] if self.bias else None)

    def projections(self) -> list:
        return [self.qkv, self.out]             # q_only is a view of qkv's first rows

    def device_driven(self) -> bool:
        return True

    # ------------------------------------------------------------------- running
    def forward(self, ctx, x, cache, states) -> Delta:
        if cache is None or cache.k_pool is None:
            raise RuntimeError("attention needs a cache with storage")
        table = ctx.tables[cache.group]
        q_cols = self.heads * self.head_dim
        rot = self.rot
        mixed = ctx.scratch("attention.mixed", (ctx.n_tokens, q_cols))
        if (cache.writes and not ctx.decode and x.dtype == torch.bfloat16
                and api.gemm_tcgen05_qkv_rope_takes(x, self.qkv.weight, self.head_dim, rot.rotary_dim)):
            # long prompts: the qkv product's epilogue rotates, narrows and appends to the cache, so the float32
            # product never goes to memory and back; positions, block lookups' inputs and the cosines and sines
            # are the same for every layer and are made once per step
            cos_sin, where = self.step_rope_table(ctx)
            q = ctx.scratch("attention.q", (ctx.n_tokens, q_cols))
            api.set_label("attention.qkv")
            api.gemm_tcgen05_qkv_rope(x, self.qkv.weight, self.qkv.bias, q, cache.k_pool, cache.v_pool, cos_sin, where, table, self.heads,
                                      self.kv_heads, self.head_dim, rot.attention_scaling, ctx.status)
            self.attend(ctx, q, cache, table, mixed)
            return self.out.delta(ctx, mixed, "attention.out")
        projection = (self.qkv if cache.writes else self.q_only)(ctx, x, "attention.qkv")
        splits = self.decode_slices(ctx)
        if (ctx.decode and ctx.sequences * self.kv_heads * splits <= api.sm_count(x.device)
                and api.attention_decode_rope_supports(mixed.dtype, self.heads, self.kv_heads, self.head_dim, rot.rotary_dim)):
            # decoding: rotation, cache write and attention in one kernel.  Every CTA pays the
            # rotation's latency before it can start on its keys, which is hidden while all CTAs
            # run at once (measured on a B200: 2 % faster at 32 and at 64 CTAs, 8 % slower at 512).
            part_acc, part_ml = self.slice_scratch(ctx, splits)
            api.attention_decode_rope(projection, rot.inv_freq, rot.rotary_dim, rot.attention_scaling, cache.writes,
                                      cache.k_pool, cache.v_pool, table, ctx.len_before, ctx.sequences, self.heads, self.kv_heads,
                                      self.head_dim, self.scale, self.window or 0, splits, mixed, part_acc, part_ml, ctx.status,
                                      tickets=self.tickets(ctx, splits))
            return self.out.delta(ctx, mixed, "attention.out")
        q = ctx.scratch("attention.q", (ctx.n_tokens, q_cols))
        api.rope_append(projection, rot.inv_freq, rot.rotary_dim, rot.attention_scaling, q,
                        cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None, table, ctx.cu,
                        ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads, self.kv_heads, self.head_dim, ctx.status)
        self.attend(ctx, q, cache, table, mixed)
        return self.out.delta(ctx, mixed, "attention.out")

    def step_rope_table(self, ctx):
        """(cos_sin, where) of this step for this layer's rotary table: made by the first layer that asks and kept
        in ``ctx.memo`` for the layers that share the table."""
        rot = self.rot
        key = ("rope_table", rot.signature or rot.inv_freq.data_ptr(), rot.rotary_dim)       # the model's layers usually share one table
        made = ctx.memo.get(key)
        if made is None:
            half = rot.rotary_dim // 2
            cos_sin = ctx.scratch(f"attention.rope_table.{len(ctx.memo)}", (ctx.n_tokens, half, 2), torch.float32)
            where = ctx.scratch(f"attention.rope_where.{len(ctx.memo)}", (ctx.n_tokens, 2), torch.int32)
            api.rope_table(rot.inv_freq, rot.rotary_dim, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, cos_sin, where)
            made = ctx.memo[key] = (cos_sin, where)
        return made

    def decode_slices(self, ctx) -> int:
        """Slices of the keys for the tensor-core decode kernel, which runs one CTA per (sequence, kv
        head, slice).  Measured on a B200 from 1 to 64 sequences and 2,048 to 32,768 keys: a step is
        fastest when the slices just fill one wave of one CTA per SM and keep at least 8 blocks each; a
        second wave gains nothing."""
        return kv_splits(ctx, ctx.sequences * self.kv_heads, 512, api.sm_count(ctx.status.device))

    def slice_scratch(self, ctx, splits: int):
        """Where the slices of the keys leave their partial results (nothing for one slice)."""
        if splits <= 1:
            return None, None
        return (ctx.scratch("attention.part_acc", (ctx.n_tokens * self.heads * splits * self.head_dim,), torch.float32),
                ctx.scratch("attention.part_ml", (ctx.n_tokens * self.heads * splits * 2,), torch.float32))

    def tickets(self, ctx, splits: int):
        """With more key slices than a thread-block cluster combines (8), the decode kernel's CTAs draw tickets and
        the last one of a (sequence, kv head) combines the slices: one word each, zero between launches."""
        if splits <= 8:
            return None
        return ctx.workspace.get_zeroed("attention.tickets", (max(ctx.sequences * self.kv_heads, 64),), torch.int32)

    def attend(self, ctx, q, cache, table, mixed) -> None:
        """Prompts in bfloat16 with head size 64 or 128: the tcgen05 kernel.  Other bfloat16
        sizes up to 128 and all decoding: the mma.sync kernels.  Everything else (float32,
        head sizes 48, 80, 144 ...): the exact kernel."""
        if not ctx.decode and api.attention_tcgen05_supports(q.dtype, self.heads, self.kv_heads, self.head_dim):
            api.attention_tcgen05(q, cache.k_pool, cache.v_pool, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads,
                                  self.kv_heads, self.head_dim, self.scale, self.window or 0, mixed, ctx.status)
            return
        tensor_cores = api.attention_mma_supports(q.dtype, self.heads, self.kv_heads, self.head_dim)
        if tensor_cores:
            splits = self.decode_slices(ctx)
        else:
            splits = kv_splits(ctx, ctx.n_tokens * self.heads, 256, 8 * api.sm_count(q.device))
        part_acc, part_ml = self.slice_scratch(ctx, splits)
        if tensor_cores:
            api.attention_mma(q, cache.k_pool, cache.v_pool, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads,
                              self.kv_heads, self.head_dim, self.scale, self.window or 0, splits, mixed, part_acc, part_ml, ctx.status,
                              one_token_each=ctx.decode, tickets=self.tickets(ctx, splits) if ctx.decode else None)
        else:
            api.attention(q, cache.k_pool, cache.v_pool, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads,
                          self.kv_heads, self.head_dim, self.scale, self.window or 0, splits, mixed, part_acc, part_ml, ctx.status)

"""A model built from a :class:`~thintensor_b200.parts.spec.ModelSpec`.

The class knows nothing of any architecture: it builds the parts the spec names from
the part registries, collects the tensors they declare under their checkpoint names,
hands each part its tensors, tells the cache what every run of the schedule needs, and
runs the schedule.  The reference's counterpart is the layer loop of
ThinGpuCausalLMRuntime (thinruntime/gpu_runtime.py:10114-10392) driven by its
execution plan.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.cache import SequenceCache
from ..parts import ARRANGEMENTS, EMBEDDINGS, HEADS, NORMS, REGISTRIES
from ..parts.base import Delta, Part, WeightDecl
from ..parts.spec import ModelSpec, PartSpec
from .context import StepContext


@dataclass
class BuiltPart:
    part: Part
    prefix: str


def _build(role_registry, spec: PartSpec) -> BuiltPart:
    return BuiltPart(role_registry.build(spec.kind, dict(spec.params)), spec.prefix)


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str | None):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.embedding = _build(EMBEDDINGS, spec.embedding)
        self.final_norm = _build(NORMS, spec.final_norm)
        self.head = _build(HEADS, spec.head)
        self.layers = []
        self._layer_parts: list[dict[str, BuiltPart]] = []
        for layer in spec.layers:
            arrangement_cls = ARRANGEMENTS._classes.get(layer.arrangement)
            if arrangement_cls is None:
                raise KeyError(f"no arrangement of kind {layer.arrangement!r}; registered: {', '.join(ARRANGEMENTS.kinds())}")
            built: dict[str, BuiltPart] = {}
            for role, registry_name in arrangement_cls.roles.items():
                if role not in layer.parts:
                    raise ValueError(f"arrangement {layer.arrangement!r} needs a part for role {role!r}")
                built[role] = _build(REGISTRIES[registry_name], layer.parts[role])
            self._layer_parts.append(built)
            self.layers.append(arrangement_cls({role: b.part for role, b in built.items()}))
        self.bound = False
        self.device_driven = False
        self.cache_needs()          # sets self.users

    # ------------------------------------------------------------------ weights
    def _all_parts(self) -> list[BuiltPart]:
        parts = [self.embedding]
        for built in self._layer_parts:
            parts.extend(built.values())
        parts.extend([self.final_norm, self.head])
        return parts

    def weight_declarations(self) -> dict[str, WeightDecl]:
        """Checkpoint name -> declaration, in the order the tensors are stored."""
        out: dict[str, WeightDecl] = {}
        for built in self._all_parts():
            for local, decl in built.part.weights().items():
                name = built.prefix + local
                if name in out and out[name] != decl:
                    raise ValueError(f"tensor {name!r} is declared twice with different shapes")
                out[name] = decl
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Give every part its tensors; ``tensors`` maps checkpoint names to device
        tensors (an aliased tensor appears under the name of its source)."""
        for built in self._all_parts():
            mine: dict[str, torch.Tensor] = {}
            for local, decl in built.part.weights().items():
                name = built.prefix + local
                if decl.alias_of is not None and (decl.prefer_alias or name not in tensors):
                    name = decl.alias_of
                if name in tensors:
                    mine[local] = tensors[name]
                elif not decl.optional:
                    raise KeyError(f"tensor {name!r} was not loaded")
            built.part.bind(mine, self.dtype, self.device)
        self.bound = True
        # a step of a shape that has run before may be replayed from a CUDA graph if no part computes on the host
        self.device_driven = all(b.part.device_driven() for b in (self.embedding, self.final_norm, self.head)) and all(
            layer.device_driven() for layer in self.layers)

    # -------------------------------------------------------------------- cache
    def cache_needs(self):
        """What the cache must hold, one entry for every mixer of every run of the schedule (in
        schedule order; a layer's mixers in the order its arrangement lists them): keys and values,
        state tensors, and the entry whose keys this one reads instead of keeping its own.  Also
        sets ``self.users``: for each run, the entries of its mixers."""
        kv, state, source = [], [], []
        self.users: list[list[int]] = []
        for run in self.spec.schedule:
            mixers = self.layers[run.layer].mixers()
            mine = list(range(len(kv), len(kv) + len(mixers)))
            if run.cache_from is not None and len(self.users[run.cache_from]) != len(mixers):
                raise ValueError(f"a run of layer {run.layer} reads the cache of a run with another number of mixers")
            for i, mixer in enumerate(mixers):
                need = mixer.cache_need()
                kv.append(need)
                state.append(list(mixer.state_needs()))
                # only keys are shared: a mixer without keys has nothing to read there, and states are always a run's own
                source.append(None if run.cache_from is None or need is None else self.users[run.cache_from][i])
            self.users.append(mine)
        return kv, state, source

    def new_cache(self, num_blocks: int, max_slots: int, device: torch.device | str | None = "default") -> SequenceCache:
        kv, state, source = self.cache_needs()
        where = self.device if device == "default" else device
        return SequenceCache(kv, state, source, num_blocks, max_slots, self.dtype, where)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: StepContext, cache: SequenceCache, rows: torch.Tensor | None) -> torch.Tensor | None:
        """Run the packed tokens of ``ctx`` through the schedule and return float32
        logits ``[len(rows), vocab]`` at the packed token indices ``rows``.  Without ``rows`` the
        step only fills the cache: the final norm and the head (which reads every row of its
        matrix whatever the number of positions) are not run and nothing is returned."""
        if not self.bound:
            raise RuntimeError("the model has no weights yet")
        residual = ctx.scratch("model.residual", (ctx.n_tokens, self.spec.hidden_size), torch.float32)
        self.embedding.part.forward(ctx, ctx.tokens, residual)
        pending: Delta | None = None
        for index, run in enumerate(self.spec.schedule):
            users = self.users[index]
            pending = self.layers[run.layer].run(ctx, residual, pending, [cache.run_cache(u) for u in users], [cache.run_state(u) for u in users])
        if rows is None:
            return None
        wanted = ctx.scratch("model.final", (rows.numel(), self.spec.hidden_size))
        self.final_norm.part.forward(ctx, residual, pending, wanted, rows)
        return self.head.part.forward(ctx, wanted)

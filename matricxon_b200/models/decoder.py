"""A decoder assembled from a ``ModelSpec``: embedding, scheduled layers, final norm, head.

The order of execution is the spec's schedule, not the layer list: an entry names
the layer whose weights run, and either owns a cache or reads an earlier entry's.
The reference's StarCoder2 is the special case "every layer once, in order"
(app/architectures/starcoder2.py:204-233): embedding lookup (:218), the layer loop
(:220-221), the final norm on the wanted positions only (:228-230), and logits
through the tied embedding or a separate head without bias (:231-233).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_F32, PendingSum, linear
from matricxon_b200.parts.base import (
    CacheBinding,
    KVCacheRequest,
    Runtime,
    StateRequest,
    build_part,
    part_class,
)
from matricxon_b200.parts.spec import ModelSpec
from matricxon_b200.weights.loader import WeightSpec


@dataclass(frozen=True)
class CacheGroupPlan:
    """Schedule entries whose caches have the same geometry and the same lifetime rule."""

    request: KVCacheRequest
    entries: tuple[int, ...]          # schedule positions that own a cache in this group


@dataclass(frozen=True)
class CachePlan:
    groups: tuple[CacheGroupPlan, ...]
    # per schedule position: (group index, index inside the group) of the cache it uses, or None
    kv_of_entry: tuple[tuple[int, int] | None, ...]
    writes: tuple[bool, ...]
    # per schedule position: the fixed-size state it asks for, or None
    state_of_entry: tuple[StateRequest | None, ...]

    @property
    def state_bytes_per_request(self) -> int:
        total = 0
        for request in self.state_of_entry:
            if request is not None:
                count = 1
                for extent in request.shape:
                    count *= extent
                total += count * torch.empty((), dtype=request.dtype).element_size()
        return total


def model_weight_specs(spec: ModelSpec) -> list[WeightSpec]:
    """Every tensor the model expects, by name, without building anything."""
    specs = [WeightSpec(f"{spec.embedding_name}.weight", (spec.vocab_size, spec.hidden_size),
                        role="matrix", init="weight")]
    for index, layer in enumerate(spec.layers):
        prefix = f"{spec.layer_prefix}.{index}."
        specs.extend(part_class("block", layer.block).weight_specs(layer, prefix))
    specs.extend(part_class("norm", spec.final_norm.kind).weight_specs(
        spec.final_norm, f"{spec.final_norm_name}."))
    if not spec.tie_word_embeddings:
        specs.append(WeightSpec(f"{spec.head_name}.weight", (spec.vocab_size, spec.hidden_size),
                                role="matrix", init="weight"))
    if spec.head_bias:
        specs.append(WeightSpec(f"{spec.head_name}.bias", (spec.vocab_size,), role="vector", init="bias"))
    return specs


def plan_cache(spec: ModelSpec) -> CachePlan:
    groups: dict[KVCacheRequest, list[int]] = {}
    own: list[KVCacheRequest | None] = []
    states: list[StateRequest | None] = []
    for position, entry in enumerate(spec.schedule):
        mixer_spec = spec.layers[entry.layer].mixer
        mixer_cls = part_class("mixer", mixer_spec.kind)
        request = mixer_cls.cache_request(mixer_spec)
        states.append(mixer_cls.state_request(mixer_spec))
        if entry.cache_of is not None:
            source = own[entry.cache_of]
            if request is not None and source is not None and \
                    (request.num_kv_heads, request.head_dim, request.planes) != \
                    (source.num_kv_heads, source.head_dim, source.planes):
                raise ValueError(f"schedule entry {position} cannot read the cache of entry "
                                 f"{entry.cache_of}: head geometry differs")
            own.append(None)
            continue
        own.append(request)
        if request is not None:
            groups.setdefault(request, []).append(position)
    group_list = list(groups.items())
    index_of: dict[int, tuple[int, int]] = {}
    for g, (_, members) in enumerate(group_list):
        for i, position in enumerate(members):
            index_of[position] = (g, i)
    kv_of_entry = []
    writes = []
    for position, entry in enumerate(spec.schedule):
        if entry.cache_of is not None:
            kv_of_entry.append(index_of.get(entry.cache_of))
            writes.append(False)
        else:
            kv_of_entry.append(index_of.get(position))
            writes.append(True)
    return CachePlan(
        groups=tuple(CacheGroupPlan(request=r, entries=tuple(m)) for r, m in group_list),
        kv_of_entry=tuple(kv_of_entry), writes=tuple(writes), state_of_entry=tuple(states))


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime) -> None:
        self.spec = spec
        self.runtime = runtime
        self.layers = [part_class("block", layer.block)(layer, runtime, f"{spec.layer_prefix}.{index}.")
                       for index, layer in enumerate(spec.layers)]
        self.final_norm = build_part("norm", spec.final_norm, runtime, f"{spec.final_norm_name}.")
        # decode steps may be captured as CUDA graphs only if every part is stream-ordered
        self.capturable = self.final_norm.capturable and all(layer.capturable for layer in self.layers)
        self.cache_plan = plan_cache(spec)
        self.embedding: torch.Tensor | None = None
        self.head: torch.Tensor | None = None
        self.head_bias: torch.Tensor | None = None
        self.bindings: list[CacheBinding] = [CacheBinding() for _ in spec.schedule]

    def weight_specs(self) -> list[WeightSpec]:
        return model_weight_specs(self.spec)

    def load(self, fetch) -> None:
        self.embedding = fetch(f"{self.spec.embedding_name}.weight")
        for layer in self.layers:
            layer.load(fetch)
        self.final_norm.load(fetch)
        self.head = (self.embedding if self.spec.tie_word_embeddings
                     else fetch(f"{self.spec.head_name}.weight"))
        self.head_bias = fetch(f"{self.spec.head_name}.bias") if self.spec.head_bias else None

    def bind_cache(self, group_storage: list[torch.Tensor], state_storage: list[torch.Tensor | None]) -> None:
        """``group_storage[g]`` is [entries, pages, planes, kv heads, page_size, head_dim];
        ``state_storage[position]`` is [slots, *shape] or None."""
        plan = self.cache_plan
        self.bindings = []
        for position in range(len(self.spec.schedule)):
            where = plan.kv_of_entry[position]
            binding = CacheBinding(writes=plan.writes[position], state=state_storage[position])
            if where is not None:
                binding.group = where[0]
                binding.kv = group_storage[where[0]][where[1]]
            self.bindings.append(binding)

    def forward(self, ctx) -> torch.Tensor:
        """Runs the step's tokens through the schedule; returns the float32 residual stream."""
        x = ctx.hidden(self.spec.hidden_size)
        kernels.embed(ctx.token_ids, self.embedding, x, ctx.status, self.spec.embedding_scale)
        # a block may hand the next one a residual sum still to be added up (the next norm adds as it reads)
        ctx.pending_sum_wanted = True
        try:
            for position, entry in enumerate(self.spec.schedule):
                layer = self.layers[entry.layer]
                if isinstance(x, PendingSum) and not layer.takes_pending_sum:
                    x = x.tensor()
                x = layer.forward(x, ctx, self.bindings[position])
        finally:
            ctx.pending_sum_wanted = False
        return x.tensor() if isinstance(x, PendingSum) else x      # the last block's sum, added up here

    def logits(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Float32 logits [len(rows), vocab] of the residual-stream rows ``rows``."""
        normed = self.final_norm.forward(x, rows=rows)
        logits = linear(normed, self.head, self.head_bias, EPILOGUE_F32, backend=self.runtime.gemm_backend)
        if self.spec.logit_softcap is not None:
            kernels.softcap(logits, self.spec.logit_softcap)
        return logits

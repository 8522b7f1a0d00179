"""Descriptions of parts: plain data that an architecture's configuration produces.

A model is described without naming the architecture it came from: a list of
layers, each naming the kind and the constants of its mixer, feed-forward and
norms, and a schedule that says in which order layers run. The reference
passes the same constants as constructor arguments
(app/architectures/starcoder2_layers.py:34-43, app/architectures/qwen_layers.py:35-45,
app/architectures/rope.py:16); here they are data so that a layer list can mix kinds.

A spec class only needs a string attribute ``kind``; the class registered under
that kind (``parts.base.register_part``) is built from it. New kinds need no change here.

No tensor name is written in this file: what the tensors of a layer are called in a
checkpoint is the architecture's business, so every name is a field that the
architecture's configuration fills in (config/starcoder2.py for StarCoder2).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class LayerNormSpec:
    """``(x - mean) / sqrt(var + eps) * weight (+ bias)`` over the last axis."""

    size: int
    eps: float
    bias: bool = True
    kind: str = "layernorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding, halves paired as (i, i + rotary_dim/2)."""

    rotary_dim: int
    theta: float
    kind: str = "rotary_neox"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged cache.

    ``window`` is None for plain causal attention; otherwise the query at
    absolute position p sees key j iff ``j <= p and j > p - window``.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    bias: bool
    window: int | None
    scale: float
    # tensor names under the mixer's prefix, without ".weight" / ".bias": either three names (the
    # query, key and value projections as separate tensors, packed into one at load) or one name
    # (a checkpoint that stores them fused: rows of q, then k, then v), and the output projection
    projection_names: tuple[str, ...]
    output_name: str
    position: Any | None = None
    kind: str = "attention"

    def __post_init__(self) -> None:
        if len(self.projection_names) not in (1, 3):
            raise ValueError("projection_names holds three names (q, k, v) or one (fused qkv), "
                             f"not {len(self.projection_names)}")
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"{self.num_heads} attention heads are no multiple of "
                             f"{self.num_kv_heads} kv heads")
        if self.head_dim <= 0 or self.head_dim % 16 != 0 or self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is not a multiple of 16 up to 256: "
                             "no attention kernel of this engine takes it")


@dataclass(frozen=True)
class MlpSpec:
    """``down(act(up(x)))`` without a gate."""

    hidden_size: int
    intermediate_size: int
    bias: bool
    activation: str
    up_name: str                 # tensor names under the feed-forward's prefix
    down_name: str
    kind: str = "mlp"


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: which block arrangement holds which parts."""

    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    ffn_norm: Any
    # weight-name fragments under the layer's prefix ("<layer_prefix>.<index>.")
    mixer_name: str
    feed_forward_name: str
    mixer_norm_name: str
    ffn_norm_name: str
    block: str = "pre_norm_sequential"


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named by several
    entries: its weights are then shared, each execution keeps a cache of its
    own). ``cache_of`` names an earlier schedule entry whose cache this
    execution reads instead of owning one; it then writes nothing.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: Any
    tie_word_embeddings: bool
    max_position_embeddings: int
    # tensor names: "<embedding_name>.weight", "<layer_prefix>.<index>.", "<final_norm_name>.",
    # "<head_name>.weight" (read only when the head is not tied to the embedding)
    embedding_name: str
    layer_prefix: str
    final_norm_name: str
    head_name: str
    # what some architectures do around the layers (StarCoder2 does none of it): the looked-up
    # embeddings times a constant, a bias on the output head ("<head_name>.bias"), and scores
    # squashed to cap * tanh(score / cap)
    embedding_scale: float = 1.0
    head_bias: bool = False
    logit_softcap: float | None = None
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self) -> None:
        for position, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {position} names layer {entry.layer}, "
                                 f"but the model has {len(self.layers)} layers")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < position:
                    raise ValueError(f"schedule entry {position} reads the cache of entry "
                                     f"{entry.cache_of}, which does not run before it")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {position} reads the cache of entry "
                                     f"{entry.cache_of}, which owns no cache itself")


def sequential_schedule(num_layers: int) -> tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i) for i in range(num_layers))

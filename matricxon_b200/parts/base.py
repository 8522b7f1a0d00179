"""What every part is, and the registry from a spec's ``kind`` to the class that runs it.

A part is built from (spec, runtime, weight-name prefix); it declares the tensors
it wants by name and shape, receives them through ``load(fetch)``, and runs on
the tensors of a step. No part knows which model it belongs to: an architecture
is only the list of specs its configuration produces. The reference wires the
same parts by constructor arguments inside each architecture's modules
(app/architectures/starcoder2_layers.py:34-57).

Interfaces (duck-typed; these base classes state them):

  Norm.forward(x, out=None, rows=None) -> activations
      x is the float32 residual stream [tokens, hidden]; result is in the runtime dtype.
  PositionEncoding.rotate_and_store(qkv, ctx, binding, n_heads, n_kv_heads, head_dim)
      encodes q (and k) inside ``qkv`` in place and stores k, v into the bound cache pages.
  Mixer.forward(h, residual, ctx, binding) -> residual + mix(h)      (float32)
  Mixer.cache_request(spec) / Mixer.state_request(spec): what the cache manager must hold.
  FeedForward.forward(h, residual, ctx) -> residual + ffn(h)          (float32)
  Block.forward(x, ctx, binding) -> x                                  (float32)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from matricxon_b200.weights.loader import WeightSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")
_PARTS: dict[str, dict[str, type]] = {category: {} for category in CATEGORIES}


class UnknownPartError(KeyError):
    pass


def register_part(category: str, kind: str, cls: type | None = None):
    """Registers ``cls`` as the implementation of ``kind``; usable as a decorator."""
    if category not in _PARTS:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")

    def _register(target: type) -> type:
        _PARTS[category][kind] = target
        return target

    return _register(cls) if cls is not None else _register


def part_class(category: str, kind: str) -> type:
    try:
        return _PARTS[category][kind]
    except KeyError:
        raise UnknownPartError(
            f"no {category} part of kind {kind!r} is registered "
            f"(known: {sorted(_PARTS.get(category, {}))})") from None


def build_part(category: str, spec: Any, runtime: "Runtime", prefix: str):
    return part_class(category, spec.kind)(spec, runtime, prefix)


@dataclass
class Runtime:
    """What a part needs to know about where and how it runs."""

    device: torch.device
    dtype: torch.dtype                    # activations, matrices and cache: bfloat16 or float32
    page_size: int = 16
    gemm_backend: str = "auto"            # "auto" | "simt" | "library" | "tcgen05"

    def __post_init__(self) -> None:
        self.device = torch.device(self.device)
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"runtime dtype must be float32 or bfloat16, not {self.dtype}")


@dataclass(frozen=True)
class KVCacheRequest:
    """Paged memory for one execution of a mixer: per page and KV head, ``planes`` tiles of
    ``page_size x head_dim`` elements. Attention asks for two (keys and values); a mixer that
    caches one vector per token (keys only, a shared latent) asks for one with
    ``num_kv_heads = 1`` and its vector's width as ``head_dim``. How a tile is laid out inside is
    the mixer's own business: the cache manager deals in pages, never in their contents.
    ``window`` None keeps every position; otherwise pages wholly older than the last
    ``window`` positions are given back."""

    num_kv_heads: int
    head_dim: int
    window: int | None
    planes: int = 2


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size state per request for one execution of a mixer."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheBinding:
    """What one schedule entry's mixer may touch in the cache.

    ``kv`` is [pages, planes, kv heads, page_size, head_dim] of the group ``group``; ``writes``
    is False when the entry reads another entry's cache. ``state`` is [slots, *shape].
    """

    group: int | None = None
    kv: torch.Tensor | None = None
    writes: bool = True
    state: torch.Tensor | None = None


class Part:
    # True when ``forward`` only enqueues work on the current CUDA stream (no host synchronisation,
    # no memory from outside the step's allocator): such a part can run inside a captured CUDA graph.
    # A model takes the graph path for decode steps only if every one of its parts says so; the
    # default is the safe answer for parts written elsewhere.
    capturable = False

    def __init__(self, spec: Any, runtime: Runtime, prefix: str) -> None:
        self.spec = spec
        self.runtime = runtime
        self.prefix = prefix

    @classmethod
    def weight_specs(cls, spec: Any, prefix: str) -> list[WeightSpec]:
        return []

    def load(self, fetch: Callable[[str], torch.Tensor]) -> None:
        return None


class Norm(Part):
    # True: forward_sum(pending) takes an ``ops.linear.PendingSum`` and returns (x, norm(x))
    adds_pending_sum = False

    def forward(self, x, out=None, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    # True: rotate_and_store takes ``bias=`` (the QKV product's bias, not yet added) and adds it itself,
    # which saves the product's epilogue pass where the product is the library's
    adds_bias = False

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim):
        raise NotImplementedError

    def project_rotate_store(self, h, weight, bias, ctx, binding, n_heads, n_kv_heads, head_dim):
        """Optional shortcut: the QKV product of ``h`` with ``weight`` / ``bias``, rotated and
        stored in one go. Returns the qkv tensor (its query columns rotated; keys and values
        are in the cache and need not be in it), or None when the encoding has no such kernel
        for this step; the mixer then runs the product and ``rotate_and_store``."""
        return None


class Mixer(Part):
    @classmethod
    def cache_request(cls, spec: Any) -> KVCacheRequest | None:
        return None

    @classmethod
    def state_request(cls, spec: Any) -> StateRequest | None:
        return None

    def forward(self, h, residual, ctx, binding):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, residual, ctx):
        raise NotImplementedError


class Block(Part):
    # True: forward() takes ``x`` as an ``ops.linear.PendingSum`` too, and returns one where
    # ``ctx.pending_sum_wanted`` says that the caller takes it (the model does, between such blocks)
    takes_pending_sum = False

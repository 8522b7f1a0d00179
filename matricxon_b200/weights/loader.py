"""Weights by tensor name, checked as a whole before anything is copied.

The reference copies tensor after tensor and stops at the first problem: a
missing name raises from the loader (app/gguf/loader.py:36-39), a wrong shape
surfaces from ``copy_`` (app/architectures/starcoder2.py:133-194), and tensors
the model does not use are ignored (app/gguf/loader.py:15-19). Here the whole
set is compared with what the model expects first, and ONE error lists every
missing tensor, every unexpected tensor and every wrong shape.

Precision held in memory, by the role a part gives each tensor:
  "matrix"    -> the compute dtype (bfloat16 when serving, float32 on the 32-bit path)
  "vector"    -> float32 always (norm scales and shifts, biases): a value stored in
                 32-bit keeps every bit, and a bfloat16 value widens without loss
  "int_table" -> int32
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Protocol

import torch


@dataclass(frozen=True)
class WeightSpec:
    name: str
    shape: tuple[int, ...]
    role: str = "matrix"          # "matrix" | "vector" | "int_table"
    init: str = "weight"          # "weight" | "bias" | "norm_weight" | "norm_bias" (random mode)


class TensorSource(Protocol):
    def names(self) -> list[str]: ...
    def shape(self, name: str) -> tuple[int, ...]: ...
    def read(self, name: str) -> torch.Tensor: ...


class DictSource:
    """Tensors already in memory (random weights, tests)."""

    def __init__(self, tensors: dict[str, torch.Tensor]) -> None:
        self.tensors = tensors

    def names(self) -> list[str]:
        return list(self.tensors)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.tensors[name].shape)

    def read(self, name: str) -> torch.Tensor:
        return self.tensors[name]


class WeightLoadError(ValueError):
    """The tensors offered do not match the tensors the model expects."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_kind=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = ["model weights do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, expected, found in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(expected)}, found {list(found)}")
        for name, why in self.wrong_kind:
            lines.append(f"  wrong dtype: {name} {why}")
        super().__init__("\n".join(lines))


def check_weights(specs: list[WeightSpec], source: TensorSource) -> None:
    expected = {spec.name: spec for spec in specs}
    if len(expected) != len(specs):
        seen: set[str] = set()
        dup = [s.name for s in specs if s.name in seen or seen.add(s.name)]
        raise ValueError(f"model declares a weight name twice: {dup}")
    present = set(source.names())
    missing = sorted(expected.keys() - present, key=_natural)
    unexpected = sorted(present - expected.keys(), key=_natural)
    wrong_shape = []
    wrong_kind = []
    for name in sorted(expected.keys() & present, key=_natural):
        found = tuple(source.shape(name))
        if found != tuple(expected[name].shape):
            wrong_shape.append((name, expected[name].shape, found))
        dtype = getattr(source, "dtype", None)
        if dtype is not None:
            stored = dtype(name)
            floating = stored.is_floating_point
            if expected[name].role == "int_table" and floating:
                wrong_kind.append((name, f"is {stored}, expected an integer table"))
            if expected[name].role != "int_table" and not floating:
                wrong_kind.append((name, f"is {stored}, expected floating point"))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightLoadError(missing, unexpected, wrong_shape, wrong_kind)


def _natural(name: str):
    return [int(piece) if piece.isdigit() else piece for piece in name.split(".")]


def held_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "matrix":
        return compute_dtype
    if role == "vector":
        return torch.float32
    if role == "int_table":
        return torch.int32
    raise ValueError(f"unknown weight role {role!r}")


def make_fetcher(specs: list[WeightSpec], source: TensorSource, compute_dtype: torch.dtype,
                 device: torch.device | str) -> Callable[[str], torch.Tensor]:
    """Checks the whole set, then returns ``fetch(name)``: the tensor on ``device`` in the
    dtype its role asks for. Each call reads one tensor, so parts can pack as they go."""
    check_weights(specs, source)
    roles = {spec.name: spec.role for spec in specs}

    def fetch(name: str) -> torch.Tensor:
        tensor = source.read(name)
        return tensor.to(device=device, dtype=held_dtype(roles[name], compute_dtype)).contiguous()

    return fetch

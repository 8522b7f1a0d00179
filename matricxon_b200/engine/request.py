"""Requests and results under the reference's names (app/runtime/generation_request.py:22-41)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal, Sequence

from matricxon_b200.sampling.config import SamplingConfig


def as_token_list(input_ids) -> list[int]:
    """Token ids from a list, a tuple, or a tensor of shape (T,) or (1, T) (the reference's
    ``input_ids`` is a (1, T) tensor, app/runtime/chat_engine.py:128)."""
    if hasattr(input_ids, "tolist"):
        input_ids = input_ids.tolist()
    if input_ids and isinstance(input_ids[0], (list, tuple)):
        if len(input_ids) != 1:
            raise ValueError("input_ids holds more than one sequence; submit one request each")
        input_ids = input_ids[0]
    return [int(token) for token in input_ids]


@dataclass(frozen=True)
class GenerationRequest:
    input_ids: Sequence[int]
    sampling: SamplingConfig = field(default_factory=SamplingConfig)


@dataclass(frozen=True)
class GenerationResult:
    token_ids: list[int]
    finish_reason: Literal["stop", "length", "cancelled", "error"]
    error: str | None = None        # what went wrong, when ``finish_reason`` is "error"

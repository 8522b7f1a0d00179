"""Sampling options under the reference's names, defaults and meanings.

Field for field the reference's ``SamplingConfig`` (app/runtime/generation_request.py:8-19):
``temperature`` (<= 0 means greedy argmax and nothing else runs, app/runtime/sampler.py:30-38),
``top_p``, ``top_k`` (0 disables), ``repeat_penalty`` (1.0 disables; applies to generated ids
only, sampler.py:12-26), ``num_ctx`` (the most tokens a request may hold), ``num_predict``
(-1: until EOS or ``num_ctx``) and ``seed`` (None: fresh entropy on every call).
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingConfig:
    temperature: float = 0.8
    top_p: float = 0.9
    top_k: int = 40
    repeat_penalty: float = 1.1
    num_ctx: int = 2048
    num_predict: int = -1
    seed: int | None = None

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0

"""Trace replay over the engine core: given token ids in, logits out, nothing sampled.

The closest thing in the reference is a test that feeds ``[PROMPT, [t], [t], [t]]`` step
by step and collects logits (tests/unit/test_fused_ops_in_models.py:16-30). This class
holds no forward pass, cache or loader of its own: it drives ``EngineCore``'s step runner,
the one generation uses.
"""

from __future__ import annotations

import torch

from matricxon_b200.engine.core import EngineCore, load_model
from matricxon_b200.engine.step import StepEntry, StepError


class TraceReplayer:
    def __init__(self, model_dir, dtype: str, max_tokens: int, page_size: int = 16,
                 device: str = "cuda:0", max_requests: int = 16, model=None,
                 poison_cache: bool = False) -> None:
        if model is None:
            _, model = load_model(model_dir, dtype=dtype, device=device, page_size=page_size)
        self.model = model
        self.core = EngineCore(model, max_cache_tokens=max_tokens, max_requests=max_requests,
                               max_step_tokens=1 << 22, poison_cache=poison_cache)

    def step(self, entries: list[dict], end: list[str]) -> torch.Tensor | None:
        """Runs one trace step; returns the wanted logits on the host (float32) or None."""
        cache = self.core.cache
        step_entries = []
        for raw in entries:
            request_id = str(raw["id"])
            tokens = [int(t) for t in raw["tokens"]]
            want = [int(w) for w in raw.get("want", [])]
            if not cache.has_request(request_id):
                cache.add_request(request_id)
            step_entries.append(StepEntry(request_id, tokens, want))
        logits = None
        if step_entries:
            device_logits = self.core.runner.run(step_entries)
            self.core.runner.check_status()
            if device_logits is not None:
                logits = device_logits.float().cpu()
        for request_id in end:
            request_id = str(request_id)
            if not cache.has_request(request_id):
                raise StepError(f"trace ends request {request_id!r}, which is not live")
            cache.free_request(request_id)
        return logits

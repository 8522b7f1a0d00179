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


class TraceFormatError(ValueError):
    """A line of a trace that is not a step as the replay program reads it."""


def parse_trace_line(line: str) -> tuple[object, list[dict], list[str]]:
    """(step, entries, end) of one line of a trace, checked: a JSON object with ``step``,
    ``entries`` (each with ``id``, a non-empty list of integer ``tokens`` and optional ``want``
    indices into them) and optional ``end`` (request ids). One error names what is wrong."""
    import json

    try:
        record = json.loads(line)
    except json.JSONDecodeError as error:
        raise TraceFormatError(f"not JSON: {error}") from None
    if not isinstance(record, dict) or "step" not in record:
        raise TraceFormatError('a step is an object with "step", "entries" and "end"')
    entries = record.get("entries", [])
    end = record.get("end", [])
    if not isinstance(entries, list) or not isinstance(end, list):
        raise TraceFormatError('"entries" and "end" must be lists')
    checked = []
    for position, raw in enumerate(entries):
        if not isinstance(raw, dict) or "id" not in raw or "tokens" not in raw:
            raise TraceFormatError(f'entry {position} needs "id" and "tokens"')
        tokens, want = raw["tokens"], raw.get("want", [])
        if not isinstance(tokens, list) or not tokens or \
                any(isinstance(t, bool) or not isinstance(t, int) for t in tokens):
            raise TraceFormatError(f"entry {position}: tokens must be a non-empty list of integers")
        if not isinstance(want, list) or any(isinstance(w, bool) or not isinstance(w, int) for w in want):
            raise TraceFormatError(f"entry {position}: want must be a list of integers")
        checked.append({"id": str(raw["id"]), "tokens": tokens, "want": want})
    return record["step"], checked, [str(request_id) for request_id in end]


class TraceReplayer:
    def __init__(self, model_dir, dtype: str, max_tokens: int, page_size: int = 16,
                 device: str = "cuda:0", max_requests: int = 16, model=None,
                 poison_cache: bool = False) -> None:
        if model is None:
            _, model = load_model(model_dir, dtype=dtype, device=device, page_size=page_size)
        self.model = model
        self.core = EngineCore(model, max_cache_tokens=max_tokens, max_requests=max_requests,
                               max_step_tokens=1 << 22, poison_cache=poison_cache)
        self.last_rows: list[tuple[str, int]] = []     # (request, absolute position) of the latest logits
        self.last_pages: dict = {}

    def step(self, entries: list[dict], end: list[str]) -> torch.Tensor | None:
        """Runs one trace step; returns the wanted logits on the host (float32) or None."""
        cache = self.core.cache
        step_entries = []
        added = []
        self.last_rows = []
        for raw in entries:
            request_id = str(raw["id"])
            tokens = [int(t) for t in raw["tokens"]]
            want = [int(w) for w in raw.get("want", [])]
            if not cache.has_request(request_id):
                cache.add_request(request_id)
                added.append(request_id)
            start = cache.record(request_id).length
            self.last_rows.extend((request_id, start + w) for w in want)
            step_entries.append(StepEntry(request_id, tokens, want))
        logits = None
        if step_entries:
            try:
                device_logits = self.core.runner.run(step_entries)
            except Exception:
                for request_id in added:          # a step that did not run leaves no request behind
                    if cache.has_request(request_id):
                        cache.free_request(request_id)
                raise
            self.core.runner.check_status()
            if device_logits is not None:
                logits = device_logits.float().cpu()
        self.last_pages = self.page_report()
        for request_id in end:
            request_id = str(request_id)
            if not cache.has_request(request_id):
                raise StepError(f"trace ends request {request_id!r}, which is not live")
            cache.free_request(request_id)
        return logits

    def page_report(self) -> dict:
        """Where the cache stands after the step's tokens were committed and before its ``end``
        requests are given back: per group the free pages, per live request its committed length
        and the physical pages it holds (in logical order, -1 where a window has given one back),
        and how many allocations so far handed out a page that somebody had held before."""
        cache = self.core.cache
        return {"page_size": cache.page_size,
                "free": cache.free_pages(),
                "total": [pool.num_pages for pool in cache.pools],
                "reused": cache.pages_reused,
                "requests": {request_id: {"length": record.length,
                                          "pages": [list(table) for table in record.tables]}
                             for request_id, record in cache.requests.items()}}

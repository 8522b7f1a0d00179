"""The Python entry point: prompts in, generated token ids out.

Named and shaped after the reference's ``ChatEngine`` (app/runtime/chat_engine.py:17-210):
``ChatEngine(model, eos_token_ids)``, ``generate(GenerationRequest) -> GenerationResult``,
``stream(request)`` yielding token ids. Where the reference runs one request per call and
leaves batching to its worker thread (app/models/worker.py:148-183), this engine owns the
scheduler: ``generate_batch`` and the ``add_request`` / ``step`` pair run many requests
through shared steps, prompt portions beside decode tokens.
"""

from __future__ import annotations

import itertools
import os
from pathlib import Path
from typing import Iterable, Iterator

from matricxon_b200.engine.core import EngineCore, load_model
from matricxon_b200.engine.request import GenerationRequest, GenerationResult, as_token_list
from matricxon_b200.engine.scheduler import FINISHED, RUNNING, Scheduler, SchedulerConfig, Sequence
from matricxon_b200.engine.step import StepEntry
from matricxon_b200.sampling.config import SamplingConfig
from matricxon_b200.sampling.sampler import BatchSampler


class ChatEngine:
    """``model`` is a model folder (config.json + model.safetensors) or a model built by
    ``matricxon_b200.engine.core`` (for instance from random weights in memory)."""

    def __init__(self, model, eos_token_ids: Iterable[int] = (), dtype: str = "bfloat16",
                 device: str = "cuda:0", max_cache_tokens: int | None = None, max_active: int = 8,
                 max_batched_tokens: int = 2048, prefill_chunk: int = 256,
                 max_model_len: int | None = None, page_size: int = 16,
                 gemm_backend: str = "auto", use_graphs: bool = True,
                 look_ahead: bool | None = None) -> None:
        if isinstance(model, (str, Path)):
            _, model = load_model(model, dtype=dtype, device=device, page_size=page_size,
                                  gemm_backend=gemm_backend)
        self.model = model
        limit = max_model_len or model.spec.max_position_embeddings
        if max_cache_tokens is None:
            max_cache_tokens = max_active * limit
        self.core = EngineCore(model, max_cache_tokens=max_cache_tokens, max_requests=max_active,
                               max_step_tokens=max(max_batched_tokens, 1), max_model_len=limit,
                               use_graphs=use_graphs)
        self.scheduler = Scheduler(
            self.core.cache,
            SchedulerConfig(max_num_seqs=max_active, max_num_batched_tokens=max_batched_tokens,
                            prefill_chunk=prefill_chunk, max_model_len=limit),
            set(eos_token_ids))
        self.sampler = BatchSampler(model.runtime.device, model.spec.vocab_size)
        self._ids = itertools.count()
        self.steps = 0
        if look_ahead is None:
            look_ahead = os.environ.get("MATRICXON_LOOK_AHEAD", "1") != "0"
        self.look_ahead = look_ahead
        self.steps_ahead = 0            # steps queued before the ids of the step before were read
        self._ahead = None              # the step queued on the device whose ids the host has not read

    # ------------------------------------------------------------------ low level
    def add_request(self, input_ids, sampling: SamplingConfig | None = None,
                    request_id: str | None = None) -> str:
        request_id = request_id if request_id is not None else f"req-{next(self._ids)}"
        self.scheduler.add(request_id, as_token_list(input_ids), sampling or SamplingConfig())
        return request_id

    def cancel(self, request_id: str) -> bool:
        return self.scheduler.cancel(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    def _launch(self, plan, before=None):
        """Queues the step of ``plan`` and its sampling on the device; returns what ``step`` needs to
        finish it later. ``before``: the launched step whose ids are this step's tokens (a step planned
        ahead): they are taken on the device, the host has not read them yet."""
        entries = []
        samplers = []
        for planned in plan.entries:
            tokens = [0] if planned.ahead else planned.sequence.token_slice(planned.start, planned.count)
            samples = planned.samples
            entries.append(StepEntry(planned.sequence.request_id, tokens,
                                     [planned.count - 1] if samples else []))
            if samples:
                samplers.append(planned.sequence.sampler)
        feed = before[2] if before is not None else None
        logits = self.core.runner.run(entries, token_feed=feed)
        handle = None
        if samplers:
            # the status word travels with the step; reading the sampled ids synchronises for both
            self.core.runner.enqueue_status_read()
            handle = self.sampler.launch(logits, samplers, pending=feed)
        ids = self.sampler.device_ids() if samplers else None
        return plan, handle, ids, entries

    def step(self) -> list[tuple[str, int, bool]]:
        """One scheduled step. Returns (request id, new token, finished) for every request
        that produced a token.

        While every running request decodes, the step after this one is queued on the device
        before this one's ids are read (``Scheduler.plan_ahead``): its token ids come from this
        step's sampler on the device, so the host's work between two steps runs beside the GPU.
        A request that stops at a token of this step has a wasted row in the step ahead; nothing
        else differs from deciding step by step."""
        launched = self._ahead
        self._ahead = None
        if launched is not None and all(e.sequence.status != RUNNING for e in launched[0].entries):
            launched = None                       # everybody in it has stopped since: nothing to collect
        if launched is None:
            plan = self.scheduler.schedule()
            if not plan.entries:
                return []
            launched = self._launch(plan)
        plan, handle, _ids, entries = launched
        if self.look_ahead and handle is not None:
            ahead = self.scheduler.plan_ahead(plan)
            if ahead is not None:
                ahead_entries = [StepEntry(e.sequence.request_id, [0], [0]) for e in ahead.entries]
                if self.core.runner.can_feed_from_device(ahead_entries):
                    self._ahead = self._launch(ahead, before=launched)
                    self.steps_ahead += 1
        if handle is not None:
            sampled = self.sampler.read(handle)
            self.core.runner.check_status(synchronised=True)
        else:
            sampled = []
            self.core.runner.check_status()
        produced = self.scheduler.step_done(plan, sampled)
        self.steps += 1
        return [(seq.request_id, token, seq.status == FINISHED) for seq, token in produced]

    def result(self, request_id: str) -> GenerationResult:
        sequence: Sequence = self.scheduler.finished.pop(request_id)
        return GenerationResult(token_ids=list(sequence.outputs),
                                finish_reason=sequence.finish_reason)

    # ------------------------------------------------------------------ the reference's calls
    def stream(self, request: GenerationRequest) -> Iterator[int]:
        """Yields one generated token id at a time (app/runtime/chat_engine.py:83-107)."""
        request_id = self.add_request(request.input_ids, request.sampling)
        try:
            while request_id not in self.scheduler.finished:
                for rid, token, _ in self.step():
                    if rid == request_id:
                        yield token
        finally:
            if request_id not in self.scheduler.finished:
                self.cancel(request_id)
            self.scheduler.finished.pop(request_id, None)

    def generate(self, request: GenerationRequest) -> GenerationResult:
        """Runs one request to its end (app/runtime/chat_engine.py:207-210)."""
        return self.generate_batch([request])[0]

    def generate_batch(self, requests: list[GenerationRequest]) -> list[GenerationResult]:
        """Runs the requests together through shared steps; results in the order given."""
        ids = [self.add_request(r.input_ids, r.sampling) for r in requests]
        while any(rid not in self.scheduler.finished for rid in ids):
            self.step()
        return [self.result(rid) for rid in ids]

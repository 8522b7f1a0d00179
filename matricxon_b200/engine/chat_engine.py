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
from matricxon_b200.engine.scheduler import (
    FINISHED,
    RUNNING,
    RequestRefused,
    Scheduler,
    SchedulerConfig,
    Sequence,
)
from matricxon_b200.engine.step import StepEntry, StepError
from matricxon_b200.sampling.config import SamplingConfig
from matricxon_b200.sampling.sampler import BatchSampler


class ChatEngine:
    """``model`` is a model folder (config.json + model.safetensors) or a model built by
    ``matricxon_b200.engine.core`` (for instance from random weights in memory)."""

    def __init__(self, model, eos_token_ids: Iterable[int] = (), dtype: str = "bfloat16",
                 device: str = "cuda:0", max_cache_tokens: int | None = None, max_active: int = 8,
                 max_batched_tokens: int = 2048, prefill_chunk: int = 512,
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
        tokens = as_token_list(input_ids)
        vocab = self.model.spec.vocab_size
        if tokens and not (0 <= min(tokens) and max(tokens) < vocab):
            raise RequestRefused(f"the prompt holds a token id outside the vocabulary of {vocab}")
        if request_id in self.scheduler.finished or self.core.cache.has_request(request_id) \
                or any(s.request_id == request_id for s in self.scheduler.waiting):
            raise RequestRefused(f"request id {request_id!r} is already in use")
        self.scheduler.add(request_id, tokens, sampling or SamplingConfig())
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

    def step(self) -> list[tuple[str, int | None, bool]]:
        """One scheduled step. Returns (request id, new token, finished) for every request that
        produced a token, and (request id, None, True) for a request that ended without one (a
        faulty step, or the end of what the pool can hold).

        While every running request decodes, the step after this one is queued on the device
        before this one's ids are read (``Scheduler.plan_ahead``): its token ids come from this
        step's sampler on the device, so the host's work between two steps runs beside the GPU.
        A request that stops at a token of this step has a wasted row in the step ahead; nothing
        else differs from deciding step by step.

        A step that fails is void for the requests at fault, and the others go on: an entry the
        host can see to be malformed (a token id outside the vocabulary, ...) ends its own request
        with ``finish_reason="error"`` before anything is launched, and the rest of the plan runs
        in the next step; a fault that only a kernel saw cannot be pinned on one request, so every
        request of that step ends with ``error`` (the reference hands the exception of a failed
        batch to every reply in it, app/runtime/batch_decode.py:82-83,101-105) and requests outside
        the step are untouched. Raises ``SchedulerStalled`` rather than returning nothing for ever
        when requests are left and none can run."""
        ended_before = set(self.scheduler.finished)
        launched = self._ahead
        self._ahead = None
        if launched is not None and all(e.sequence.status != RUNNING for e in launched[0].entries):
            launched = None                       # everybody in it has stopped since: nothing to collect
        if launched is None:
            plan = self.scheduler.schedule()
            if not plan.entries:
                return self._ended_since(ended_before, [])
            try:
                launched = self._launch(plan)
            except StepError as error:
                if not error.request_ids:
                    raise
                for planned in plan.entries:
                    if planned.sequence.request_id in error.request_ids:
                        self.scheduler.fail(planned.sequence, str(error))
                return self._ended_since(ended_before, [])
        plan, handle, _ids, entries = launched
        if self.look_ahead and handle is not None:
            ahead = self.scheduler.plan_ahead(plan)
            if ahead is not None:
                ahead_entries = [StepEntry(e.sequence.request_id, [0], [0]) for e in ahead.entries]
                if self.core.runner.can_feed_from_device(ahead_entries):
                    self._ahead = self._launch(ahead, before=launched)
                    self.steps_ahead += 1
        try:
            if handle is not None:
                sampled = self.sampler.read(handle)
                self.core.runner.check_status(synchronised=True)
            else:
                sampled = []
                self.core.runner.check_status()
        except StepError as error:
            # a kernel met a bad index: what the step wrote and chose is void for all its requests,
            # and so is the step queued behind it, which holds the same requests
            self._ahead = None
            for planned in plan.entries:
                if planned.sequence.status == RUNNING:
                    self.scheduler.fail(planned.sequence, str(error))
            self.steps += 1
            return self._ended_since(ended_before, [])
        produced = self.scheduler.step_done(plan, sampled)
        self.steps += 1
        return self._ended_since(
            ended_before, [(seq.request_id, token, seq.status == FINISHED) for seq, token in produced])

    def _ended_since(self, before: set, produced: list) -> list:
        """``produced`` plus (id, None, True) for requests that ended during this call without a token."""
        with_token = {rid for rid, _, _ in produced}
        silent = [rid for rid in self.scheduler.finished if rid not in before and rid not in with_token]
        return produced + [(rid, None, True) for rid in silent]

    def result(self, request_id: str) -> GenerationResult:
        sequence: Sequence = self.scheduler.finished.pop(request_id)
        return GenerationResult(token_ids=list(sequence.outputs),
                                finish_reason=sequence.finish_reason, error=sequence.error)

    # ------------------------------------------------------------------ the reference's calls
    def stream(self, request: GenerationRequest) -> Iterator[int]:
        """Yields one generated token id at a time (app/runtime/chat_engine.py:83-107)."""
        request_id = self.add_request(request.input_ids, request.sampling)
        try:
            while request_id not in self.scheduler.finished:
                for rid, token, _ in self.step():
                    if rid == request_id and token is not None:
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

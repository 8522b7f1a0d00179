"""Which requests run in the next step, with how many tokens each.

The reference's worker admits replies in arrival order up to ``max_active``
(app/models/worker.py:164-172), advances every prefilling reply by one 256-token piece per
round and then runs one batched decode (worker.py:177-179; app/runtime/chat_engine.py:36,
158-182), finishes on an EOS token (which is emitted) or after ``num_predict`` tokens bounded
by ``num_ctx`` (chat_engine.py:153-154,191-196), and can never run out of cache because each
request's cache is allocated whole up front (app/runtime/kv_cache.py:31-38).

Here one step holds decode tokens and prompt portions together, under a token budget:
  1. every running request that has one token left to compute (a decode) gets it first;
  2. the rest of the budget goes to prompt portions, running requests before waiting ones,
     in arrival order, each at most ``prefill_chunk`` tokens and cut to the remaining budget;
  3. waiting requests are admitted while fewer than ``max_num_seqs`` run and pages are free.
When pages run out: portions are cut (halved until they fit) or wait while something else in
the step moves; a decode token that cannot get its page, or the oldest prompt portion when
nothing else moves, makes the most recently admitted running request give up its pages
(never an older one: the youngest gives way itself). A preempted request keeps its sampled
tokens, returns to the front of the queue and is later recomputed as one prompt of
(prompt + sampled tokens). Its random stream is a function of (seed, token index), so the
tokens it goes on to sample are unchanged. The oldest running request therefore always
advances, which is why every request ends (the property the reference's worker has by
construction: tests/unit/test_batching_scheduler.py:44-60,153-176). A request alone that
still cannot get a page ends with ``length``; one that cannot fit in the empty pool is
refused when it is added.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from matricxon_b200.cache.manager import CacheManager
from matricxon_b200.sampling.config import SamplingConfig
from matricxon_b200.sampling.sampler import RequestSampler

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class RequestRefused(ValueError):
    """A request that can never run under the engine's limits."""


class SchedulerStalled(RuntimeError):
    """Requests are left, none of them can run, and nothing is in flight that would change that."""


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 8                  # the reference's max_active default (app/config.py:87)
    max_num_batched_tokens: int = 2048
    # The reference cuts prompts into pieces of 256 tokens (PLAIN_PREFILL_CHUNK, app/runtime/chat_engine.py:36).
    # Here every step is a pass over all weights, so short pieces are dear: measured at StarCoder2-3B
    # sizes a step costs 16 us a token at 256 tokens, 10 at 512 and 6 at 1,024-2,048, while the requests
    # decoding beside a 512-token piece wait about 5 ms for their next token instead of 2.
    prefill_chunk: int = 512
    max_model_len: int = 4096


@dataclass(eq=False)
class Sequence:
    request_id: str
    prompt: list[int]
    sampling: SamplingConfig
    max_new_tokens: int
    sampler: RequestSampler
    outputs: list[int] = field(default_factory=list)
    computed: int = 0                      # tokens of prompt + outputs already in the cache
    status: str = WAITING
    finish_reason: str | None = None
    preemptions: int = 0
    order: int = 0                         # admission order among running requests
    error: str | None = None               # why, when ``finish_reason`` is "error"

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.outputs

    def token_slice(self, start: int, count: int) -> list[int]:
        """Tokens [start, start + count) of prompt + outputs without joining the two lists."""
        n_prompt = len(self.prompt)
        if start >= n_prompt:
            return self.outputs[start - n_prompt:start - n_prompt + count]
        if start + count <= n_prompt:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.outputs[:start + count - n_prompt]

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.outputs) - self.computed


@dataclass
class PlannedEntry:
    sequence: Sequence
    start: int
    count: int
    ahead: bool = False        # planned before the token of the step before it was known (``plan_ahead``)

    @property
    def samples(self) -> bool:
        """The portion reaches the request's last token: its logits choose the next one."""
        seq = self.sequence
        return self.ahead or self.start + self.count == len(seq.prompt) + len(seq.outputs)


@dataclass
class StepPlan:
    entries: list[PlannedEntry] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)
    ended: int = 0             # requests that planning itself finished (``length`` at the pool's end, ``error``)

    @property
    def num_tokens(self) -> int:
        return sum(entry.count for entry in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, config: SchedulerConfig,
                 eos_token_ids: set[int] | None = None) -> None:
        self.cache = cache
        self.config = config
        self.eos_token_ids = set(eos_token_ids or ())
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.finished: dict[str, Sequence] = {}
        self._admitted = 0
        self.num_preemptions = 0

    # ------------------------------------------------------------------ requests
    def add(self, request_id: str, prompt: list[int], sampling: SamplingConfig) -> Sequence:
        if not prompt:
            raise RequestRefused("a request needs at least one prompt token")
        limit = min(sampling.num_ctx, self.config.max_model_len)
        if len(prompt) > limit:
            raise RequestRefused(f"prompt of {len(prompt)} tokens exceeds the context of {limit}")
        room = max(limit - len(prompt), 0)
        max_new = room if sampling.num_predict < 0 else min(sampling.num_predict, room)
        most_pages = (len(prompt) + max_new + self.cache.page_size - 1) // self.cache.page_size
        page_size = self.cache.page_size
        for group, pool in enumerate(self.cache.pools):
            window = self.cache.rules[group].window
            need = most_pages
            if window is not None:
                # a window of W keys spans at most ceil((W - 1) / page) + 1 pages, and the next token's
                # page is taken before the oldest is given back
                need = min(most_pages, (window - 1 + page_size - 1) // page_size + 2)
            if need > pool.num_pages:
                raise RequestRefused(
                    f"request needs {need} pages in group {group}, the pool has {pool.num_pages}")
        sequence = Sequence(request_id, list(prompt), sampling, max_new, RequestSampler(sampling))
        if max_new == 0:
            sequence.status, sequence.finish_reason = FINISHED, "length"
            self.finished[request_id] = sequence
            return sequence
        self.waiting.append(sequence)
        return sequence

    def cancel(self, request_id: str) -> bool:
        """Stops a request between steps; False if it is neither waiting nor running."""
        for sequence in list(self.waiting):
            if sequence.request_id == request_id:
                self.waiting.remove(sequence)
                self._finish(sequence, "cancelled")
                return True
        for sequence in self.running:
            if sequence.request_id == request_id:
                self._finish(sequence, "cancelled")
                return True
        return False

    def fail(self, sequence: Sequence, why: str) -> None:
        """Ends a waiting or running request whose step was void; its pages go back at once."""
        if sequence.status == FINISHED:
            return
        if sequence.status == WAITING:
            self.waiting.remove(sequence)
        sequence.error = why
        self._finish(sequence, "error")

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _fits(self, sequence: Sequence, count: int, planned: list[int]) -> bool:
        needed = self.cache.pages_needed(sequence.request_id, count)
        free = self.cache.free_pages()
        return all(n + p <= f for n, p, f in zip(needed, planned, free))

    def _plan(self, plan: StepPlan, sequence: Sequence, count: int, planned: list[int]) -> None:
        for group, n in enumerate(self.cache.pages_needed(sequence.request_id, count)):
            planned[group] += n
        plan.entries.append(PlannedEntry(sequence, sequence.computed, count))

    def _preempt(self, sequence: Sequence, plan: StepPlan) -> None:
        self.cache.free_request(sequence.request_id)
        self.running.remove(sequence)
        sequence.status = WAITING
        sequence.computed = 0
        sequence.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(sequence)
        plan.preempted.append(sequence)

    def _youngest_unplanned(self, plan: StepPlan) -> Sequence | None:
        candidates = [s for s in self.running if all(e.sequence is not s for e in plan.entries)]
        return max(candidates, key=lambda s: s.order) if candidates else None

    def _make_room(self, sequence: Sequence, count: int, planned: list[int], plan: StepPlan) -> bool:
        """Preempts the most recently admitted requests that are not part of ``plan`` until
        ``sequence`` can have pages for ``count`` tokens. Older requests are never touched: when
        ``sequence`` is itself the youngest it is the one that goes (or, alone in the pool, ends
        with ``length``: it has reached what the pool can hold). True if the tokens fit now."""
        while not self._fits(sequence, count, planned):
            victim = self._youngest_unplanned(plan)
            if victim is None:
                return False
            if victim is sequence:
                if len(self.running) == 1:
                    self._finish(sequence, "length")
                else:
                    self._preempt(sequence, plan)
                return False
            self._preempt(victim, plan)
        return True

    def schedule(self) -> StepPlan:
        """The next step. Never empty while a request can move: a plan that only preempted is
        retried at once, and a state in which requests are left but none can run (which the rules
        above exclude) raises instead of returning an empty plan for ever."""
        plan = self._schedule_once()
        preempted = list(plan.preempted)
        while not plan.entries and self.has_work() and (plan.preempted or plan.ended):
            plan = self._schedule_once()
            preempted.extend(plan.preempted)
        plan.preempted = preempted
        if not plan.entries and self.has_work():
            raise SchedulerStalled(
                f"{len(self.running)} running and {len(self.waiting)} waiting requests, none can run "
                f"(free pages per group: {self.cache.free_pages()})")
        return plan

    def _schedule_once(self) -> StepPlan:
        plan = StepPlan()
        planned = [0] * len(self.cache.pools)
        budget = self.config.max_num_batched_tokens

        # 1. decode tokens, oldest request first; the youngest unplanned request goes when a page is missing
        for sequence in sorted(self.running, key=lambda s: s.order):
            if sequence.status != RUNNING or sequence.remaining != 1 or budget <= 0:
                continue
            finished_before = len(self.finished)
            if self._make_room(sequence, 1, planned, plan):
                self._plan(plan, sequence, 1, planned)
                budget -= 1
            plan.ended += len(self.finished) - finished_before

        # 2. prompt portions of running requests, in admission order
        def portion(sequence: Sequence) -> int:
            count = min(self.config.prefill_chunk, sequence.remaining, budget)
            while count > 0 and not self._fits(sequence, count, planned):
                count //= 2                    # a shorter portion may still fit the free pages
            return count

        blocked = False
        for sequence in sorted(self.running, key=lambda s: s.order):
            if sequence.status != RUNNING or sequence.remaining <= 1 \
                    or any(e.sequence is sequence for e in plan.entries):
                continue
            if budget <= 0:
                break
            count = portion(sequence)
            if count <= 0 and not plan.entries:
                # nothing else moves in this step, so nothing will free a page by itself: the
                # youngest requests give theirs up until the oldest portion has one
                finished_before = len(self.finished)
                if self._make_room(sequence, 1, planned, plan):
                    count = portion(sequence)
                plan.ended += len(self.finished) - finished_before
            if count <= 0:
                blocked = True                 # older requests move; this one waits for their pages
                break
            self._plan(plan, sequence, count, planned)
            budget -= count

        # 3. admit waiting requests in order
        while self.waiting and not blocked and budget > 0 \
                and len(self.running) < self.config.max_num_seqs:
            sequence = self.waiting[0]
            if any(s is sequence for s in plan.preempted):
                break                          # a request preempted in this step waits a step
            if self.cache.slots.free_count == 0:
                break
            self.cache.add_request(sequence.request_id)
            count = portion(sequence)
            if count <= 0:
                self.cache.free_request(sequence.request_id)
                if not self.running:
                    # not one token fits the empty pool: ``add`` refuses such requests, so this is
                    # a pool smaller than a page per group; the request ends, the others go on
                    self.waiting.popleft()
                    sequence.error = "the request does not fit in the empty cache pool"
                    self._finish(sequence, "error")
                    plan.ended += 1
                    continue
                break
            self.waiting.popleft()
            sequence.status = RUNNING
            sequence.order = self._admitted
            self._admitted += 1
            self.running.append(sequence)
            self._plan(plan, sequence, count, planned)
            budget -= count
        return plan

    def plan_ahead(self, plan: StepPlan) -> StepPlan | None:
        """The step after ``plan``, planned while ``plan`` still runs and its tokens are unknown: the
        same requests, one token further. Only when that is certainly what ``schedule`` would
        decide once the tokens are known, up to requests that stop at a token of ``plan`` (their
        rows of the step ahead are wasted and dropped by ``step_done``): every running request
        decodes in ``plan``, nobody waits, nobody reaches its length limit with the token of
        ``plan``, and every request can have one more slot of cache. Otherwise None."""
        if self.waiting or plan.preempted or not plan.entries or len(plan.entries) != len(self.running):
            return None
        ahead = StepPlan()
        planned = [0] * len(self.cache.pools)
        for entry in plan.entries:
            sequence = entry.sequence
            if (entry.count != 1 or not entry.samples or sequence.status != RUNNING
                    or len(sequence.outputs) + 2 > sequence.max_new_tokens
                    or not self._fits(sequence, 1, planned)):
                return None
            for group, n in enumerate(self.cache.pages_needed(sequence.request_id, 1)):
                planned[group] += n
            ahead.entries.append(PlannedEntry(sequence, entry.start + 1, 1, ahead=True))
        return ahead

    # ------------------------------------------------------------------ after a step
    def _finish(self, sequence: Sequence, reason: str) -> None:
        if sequence.status == RUNNING:
            self.cache.free_request(sequence.request_id)
            self.running.remove(sequence)
        sequence.status, sequence.finish_reason = FINISHED, reason
        self.finished[sequence.request_id] = sequence

    def step_done(self, plan: StepPlan, sampled: list[int]) -> list[tuple[Sequence, int]]:
        """Records a finished step: ``sampled`` holds one token per sampling entry, in plan
        order. Returns (sequence, new token) pairs; finished requests have given up their
        pages when this returns."""
        produced: list[tuple[Sequence, int]] = []
        tokens = iter(sampled)
        for entry in plan.entries:
            sequence = entry.sequence
            samples = entry.samples
            sequence.computed = entry.start + entry.count
            if not samples:
                continue
            token = int(next(tokens))
            if sequence.status != RUNNING:
                continue                       # cancelled while the step ran
            sequence.outputs.append(token)
            sequence.sampler.accept(token)
            produced.append((sequence, token))
            if token in self.eos_token_ids:
                self._finish(sequence, "stop")
            elif len(sequence.outputs) >= sequence.max_new_tokens:
                self._finish(sequence, "length")
        return produced

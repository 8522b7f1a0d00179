"""The scheduler's decisions with a fake step function (no GPU), in the manner of the
reference's scheduler tests with a fake decoder (tests/unit/test_batching_scheduler.py:14-23)."""

import pytest

from matricxon_b200.cache.manager import CacheManager, GroupRule
from matricxon_b200.engine.scheduler import (
    FINISHED,
    RUNNING,
    RequestRefused,
    Scheduler,
    SchedulerConfig,
)
from matricxon_b200.sampling.config import SamplingConfig
from matricxon_b200.sampling.sampler import uniform_for


def make(pages=64, page_size=4, window=None, eos=(), **config):
    cache = CacheManager([GroupRule(window)], pages, page_size, num_state_slots=8)
    defaults = dict(max_num_seqs=4, max_num_batched_tokens=16, prefill_chunk=8, max_model_len=256)
    defaults.update(config)
    return cache, Scheduler(cache, SchedulerConfig(**defaults), set(eos))


def fake_token(sequence, upto):
    """What a model would 'predict' after ``upto`` tokens: a function of the tokens alone."""
    tokens = sequence.tokens[:upto]
    return (sum((i + 1) * t for i, t in enumerate(tokens)) + len(tokens)) % 50 + 3


def run_step(cache, scheduler, log=None):
    plan = scheduler.schedule()
    sampled = []
    for entry in plan.entries:
        cache.reserve(entry.sequence.request_id, entry.count)
        cache.commit(entry.sequence.request_id, entry.count)
        if entry.samples:
            sampled.append(fake_token(entry.sequence, entry.start + entry.count))
    if log is not None:
        log.append([(e.sequence.request_id, e.start, e.count) for e in plan.entries])
    cache.check_invariants()
    return plan, scheduler.step_done(plan, sampled)


def run_all(cache, scheduler, log=None, limit=2000):
    for _ in range(limit):
        if not scheduler.has_work():
            return
        run_step(cache, scheduler, log)
    raise AssertionError("scheduler did not finish")


def sampling(num_predict=6, num_ctx=256, **kw):
    return SamplingConfig(temperature=0.0, num_predict=num_predict, num_ctx=num_ctx, **kw)


def test_single_request_prefill_in_portions_then_decode():
    cache, scheduler = make()
    scheduler.add("a", list(range(1, 21)), sampling(num_predict=3))
    log = []
    run_all(cache, scheduler, log)
    assert log[:3] == [[("a", 0, 8)], [("a", 8, 8)], [("a", 16, 4)]]      # chunk 8, then the rest
    assert log[3:] == [[("a", 20, 1)], [("a", 21, 1)]]                     # two decode steps
    done = scheduler.finished["a"]
    assert len(done.outputs) == 3 and done.finish_reason == "length"
    assert cache.free_pages() == [64]


def test_budget_decodes_first_then_portions():
    cache, scheduler = make(max_num_batched_tokens=10, prefill_chunk=8)
    scheduler.add("a", [1, 2, 3], sampling(num_predict=20))
    run_step(cache, scheduler)                                 # a: whole prompt, samples
    scheduler.add("b", list(range(1, 31)), sampling(num_predict=2))
    log = []
    run_step(cache, scheduler, log)
    assert log[0] == [("a", 3, 1), ("b", 0, 8)]                # decode first, then the portion
    scheduler.add("c", list(range(1, 31)), sampling(num_predict=2))
    run_step(cache, scheduler, log)
    # budget 10: a's decode, 8 of b, and the one token left for c
    assert log[1] == [("a", 4, 1), ("b", 8, 8), ("c", 0, 1)]
    assert sum(count for _, _, count in log[1]) == 10


def test_max_num_seqs_and_fifo_admission():
    cache, scheduler = make(max_num_seqs=2, max_num_batched_tokens=64, prefill_chunk=64)
    for name in "abc":
        scheduler.add(name, [1, 2, 3, 4], sampling(num_predict=2))
    log = []
    run_step(cache, scheduler, log)
    assert [e[0] for e in log[0]] == ["a", "b"] and len(scheduler.waiting) == 1
    run_all(cache, scheduler, log)
    assert [e[0] for e in log[2]] == ["c"]                     # admitted once a and b are done
    assert all(scheduler.finished[n].finish_reason == "length" for n in "abc")


def test_eos_is_emitted_then_stops():
    cache, scheduler = make()
    scheduler.add("probe", [5, 6, 7], sampling(num_predict=10))
    run_all(cache, scheduler)
    tokens = scheduler.finished["probe"].outputs
    cache2, scheduler2 = make(eos=[tokens[2]])
    scheduler2.add("a", [5, 6, 7], sampling(num_predict=10))
    run_all(cache2, scheduler2)
    done = scheduler2.finished["a"]
    assert done.outputs == tokens[:3] and done.finish_reason == "stop"


def test_num_ctx_bounds_generation_and_rejects_long_prompts():
    cache, scheduler = make()
    scheduler.add("a", [1] * 10, sampling(num_predict=-1, num_ctx=14))
    run_all(cache, scheduler)
    assert len(scheduler.finished["a"].outputs) == 4           # until num_ctx
    with pytest.raises(RequestRefused):
        scheduler.add("b", [1] * 15, sampling(num_ctx=14))
    with pytest.raises(RequestRefused):
        scheduler.add("c", [], sampling())
    done = scheduler.add("d", [1] * 14, sampling(num_predict=5, num_ctx=14))
    assert done.status == FINISHED and done.finish_reason == "length" and done.outputs == []
    small_cache, small = make(pages=10)
    with pytest.raises(RequestRefused):
        small.add("e", [1] * 30, SamplingConfig(num_predict=100, num_ctx=1000))   # 130 tokens > pool


def test_batched_tokens_equal_alone():
    prompts = {"a": [3, 1, 4, 1, 5], "b": list(range(2, 25)), "c": [9, 9]}
    alone = {}
    for name, prompt in prompts.items():
        cache, scheduler = make()
        scheduler.add(name, prompt, sampling(num_predict=7))
        run_all(cache, scheduler)
        alone[name] = scheduler.finished[name].outputs
    cache, scheduler = make()
    for name, prompt in prompts.items():
        scheduler.add(name, prompt, sampling(num_predict=7))
    log = []
    run_all(cache, scheduler, log)
    assert max(len(step) for step in log) >= 3
    for name in prompts:
        assert scheduler.finished[name].outputs == alone[name]


def test_pages_run_out_portions_wait_decodes_go_on():
    cache, scheduler = make(pages=6, page_size=4, max_num_batched_tokens=64, prefill_chunk=64)
    scheduler.add("a", [1] * 10, sampling(num_predict=2))      # 3 pages
    run_step(cache, scheduler)
    scheduler.add("b", [2] * 20, sampling(num_predict=2))      # 5 pages: only 3 free
    log = []
    run_step(cache, scheduler, log)
    # b is cut to the portion that fits the free pages; a decodes beside it
    assert log[0][0] == ("a", 10, 1)
    assert log[0][1][0] == "b" and log[0][1][2] < 20
    run_all(cache, scheduler, log)
    assert scheduler.finished["b"].finish_reason == "length" and cache.free_pages() == [6]


def test_preemption_keeps_tokens_and_requeues_in_front():
    prompts = {"a": [1] * 6, "b": [2] * 6, "c": [3] * 6}
    alone = {}
    for name, prompt in prompts.items():
        cache, scheduler = make()
        scheduler.add(name, prompt, sampling(num_predict=12))
        run_all(cache, scheduler)
        alone[name] = scheduler.finished[name].outputs
    # 18 tokens of prompt + 36 generated need 15 pages of 4; give 9: someone must be preempted
    cache, scheduler = make(pages=9, page_size=4, max_num_batched_tokens=64, prefill_chunk=64)
    for name, prompt in prompts.items():
        scheduler.add(name, prompt, sampling(num_predict=12))
    log = []
    preempted = []
    for _ in range(500):
        if not scheduler.has_work():
            break
        plan, _ = run_step(cache, scheduler, log)
        preempted.extend(s.request_id for s in plan.preempted)
    assert not scheduler.has_work()
    assert scheduler.num_preemptions >= 1 and preempted
    assert preempted[0] == "c"                                  # the most recently admitted goes first
    for name in prompts:
        assert scheduler.finished[name].outputs == alone[name], name
    # a recomputation runs prompt + kept tokens as one prompt
    victim = preempted[0]
    restarts = [step for step in log if any(e[0] == victim and e[1] == 0 for e in step)]
    assert len(restarts) >= 2
    assert cache.free_pages() == [9]


def test_request_alone_that_exhausts_the_pool_finishes():
    cache, scheduler = make(pages=3, page_size=4, window=None)
    scheduler.add("a", [1] * 8, sampling(num_predict=4))       # fits exactly: 12 tokens = 3 pages
    run_all(cache, scheduler)
    assert len(scheduler.finished["a"].outputs) == 4
    with pytest.raises(RequestRefused):
        scheduler.add("b", [1] * 8, sampling(num_predict=8))   # 16 tokens never fit 3 pages


def test_window_lets_a_long_request_run_in_few_pages():
    cache, scheduler = make(pages=5, page_size=4, window=8, max_num_batched_tokens=4, prefill_chunk=4)
    scheduler.add("a", [1] * 30, sampling(num_predict=20))
    run_all(cache, scheduler)
    assert len(scheduler.finished["a"].outputs) == 20
    assert cache.pages_reused > 0 and cache.free_pages() == [5]


def test_cancel_waiting_and_running():
    cache, scheduler = make(max_num_seqs=1)
    scheduler.add("a", [1, 2, 3], sampling(num_predict=50))
    scheduler.add("b", [1, 2, 3], sampling(num_predict=50))
    run_step(cache, scheduler)
    assert scheduler.cancel("b") and scheduler.finished["b"].finish_reason == "cancelled"
    assert scheduler.cancel("a") and cache.free_pages() == [64]
    assert not scheduler.cancel("a") and not scheduler.has_work()
    assert scheduler.schedule().entries == []


def test_uniform_stream_is_a_function_of_seed_and_index():
    a = [uniform_for(7, i) for i in range(50)]
    assert a == [uniform_for(7, i) for i in range(50)]
    assert a != [uniform_for(8, i) for i in range(50)]
    assert all(0.0 <= u < 1.0 for u in a) and len(set(a)) == 50
    assert abs(sum(uniform_for(1, i) for i in range(4000)) / 4000 - 0.5) < 0.02


def test_plan_ahead_only_when_the_next_step_is_certain():
    """The step planned before the tokens of the running one are known is the same requests one
    token further, and is refused whenever ``schedule`` might decide otherwise."""
    cache, scheduler = make(pages=6, page_size=4)
    scheduler.add("a", [1, 2, 3], sampling(num_predict=4))
    scheduler.add("b", [4, 5, 6, 7, 8], sampling(num_predict=9))
    plan = scheduler.schedule()
    assert scheduler.plan_ahead(plan) is None                  # prompts, not single decoded tokens
    for entry in plan.entries:
        cache.reserve(entry.sequence.request_id, entry.count)
        cache.commit(entry.sequence.request_id, entry.count)
    scheduler.step_done(plan, [9, 9])
    plan = scheduler.schedule()                                # a and b decode
    assert [(e.sequence.request_id, e.start, e.count) for e in plan.entries] == [("a", 3, 1), ("b", 5, 1)]
    for entry in plan.entries:
        cache.reserve(entry.sequence.request_id, entry.count)
        cache.commit(entry.sequence.request_id, entry.count)
    ahead = scheduler.plan_ahead(plan)
    assert [(e.sequence.request_id, e.start, e.count, e.ahead, e.samples) for e in ahead.entries] == [
        ("a", 4, 1, True, True), ("b", 6, 1, True, True)]
    scheduler.add("c", [1, 2], sampling())
    assert scheduler.plan_ahead(plan) is None                  # somebody waits: the next step may admit them
    scheduler.cancel("c")
    assert scheduler.plan_ahead(plan) is not None
    # the step ahead runs; a stops at a token of the step before it: its row of the step ahead is dropped
    for entry in ahead.entries:
        cache.reserve(entry.sequence.request_id, entry.count)
        cache.commit(entry.sequence.request_id, entry.count)
    scheduler.eos_token_ids = {33}
    assert [(s.request_id, t) for s, t in scheduler.step_done(plan, [33, 10])] == [("a", 33), ("b", 10)]
    assert scheduler.finished["a"].finish_reason == "stop"
    assert [(s.request_id, t) for s, t in scheduler.step_done(ahead, [11, 12])] == [("b", 12)]
    cache.check_invariants()
    assert scheduler.running[0].outputs == [9, 10, 12]
    # b alone: 3 + 5 tokens hold 2 pages; length limits and the pool's end refuse the step ahead
    while scheduler.has_work():
        plan = scheduler.schedule()
        for entry in plan.entries:
            cache.reserve(entry.sequence.request_id, entry.count)
            cache.commit(entry.sequence.request_id, entry.count)
        sequence = plan.entries[0].sequence
        ahead = scheduler.plan_ahead(plan)
        assert (ahead is not None) == (len(sequence.outputs) + 2 <= 9)
        scheduler.step_done(plan, [7])
    assert cache.free_pages() == [6]


def test_plan_ahead_refused_when_no_page_is_left_for_it():
    cache, scheduler = make(pages=3, page_size=4)
    scheduler.add("a", [1, 2, 3], sampling(num_predict=5))
    scheduler.add("b", [4, 5, 6], sampling(num_predict=5))
    run_step(cache, scheduler)                                 # both prompts: a page each
    plan = scheduler.schedule()                                # the fourth token of each: same pages
    assert [(e.start, e.count) for e in plan.entries] == [(3, 1), (3, 1)]
    for entry in plan.entries:
        cache.reserve(entry.sequence.request_id, 1)
        cache.commit(entry.sequence.request_id, 1)
    assert cache.free_pages() == [1]
    assert scheduler.plan_ahead(plan) is None                  # both would need a new page, one is left
    scheduler.cancel("b")
    assert scheduler.plan_ahead(plan) is None                  # the running step holds a request that left
    scheduler.step_done(plan, [5, 5])
    plan = scheduler.schedule()
    cache.reserve("a", 1)
    cache.commit("a", 1)
    assert scheduler.plan_ahead(plan) is not None


def outputs_in_roomy_pool(prompts, num_predict, **config):
    cache, scheduler = make(pages=4096, **config)
    for name, prompt in prompts.items():
        scheduler.add(name, prompt, sampling(num_predict=num_predict, num_ctx=4096))
    run_all(cache, scheduler)
    return {name: scheduler.finished[name].outputs for name in prompts}


@pytest.mark.parametrize("pages, page_size, length, chunk", [(10, 16, 100, 32), (100, 16, 960, 256)])
def test_two_prompts_that_do_not_fit_together_both_finish(pages, page_size, length, chunk):
    """Every running request is in the middle of its prompt and the pool is empty: nothing decodes,
    so nothing would ever free a page. The younger request gives way and both finish with the
    tokens they produce in a roomy pool."""
    prompts = {"a": [1 + i % 7 for i in range(length)], "b": [2 + i % 5 for i in range(length)]}
    config = dict(page_size=page_size, max_num_batched_tokens=2 * chunk, prefill_chunk=chunk,
                  max_model_len=4096)
    expected = outputs_in_roomy_pool(prompts, 4, **config)
    cache, scheduler = make(pages=pages, **config)
    for name, prompt in prompts.items():
        scheduler.add(name, prompt, sampling(num_predict=4, num_ctx=4096))
    log = []
    for _ in range(200):
        if not scheduler.has_work():
            break
        plan, _ = run_step(cache, scheduler, log)
        assert plan.entries, "an empty plan while requests are left"
    assert not scheduler.has_work()
    assert scheduler.num_preemptions >= 1
    assert {n: scheduler.finished[n].outputs for n in prompts} == expected
    assert all(scheduler.finished[n].finish_reason == "length" for n in prompts)
    assert cache.free_pages() == [pages]


def test_the_youngest_gives_way_never_an_older_request():
    """A decoding request that needs a page while an older request is still in its prompt gives up
    its own pages: the oldest running request always advances."""
    cache, scheduler = make(pages=8, page_size=4, max_num_batched_tokens=8, prefill_chunk=4)
    scheduler.add("old", [1] * 24, sampling(num_predict=2))        # 6 pages of prompt, slowly
    run_step(cache, scheduler)
    scheduler.add("young", [2] * 4, sampling(num_predict=12))      # one page, then decodes
    log, preempted = [], []
    for _ in range(100):
        if not scheduler.has_work():
            break
        plan, _ = run_step(cache, scheduler, log)
        preempted.extend(s.request_id for s in plan.preempted)
        assert plan.entries
    assert not scheduler.has_work()
    assert preempted and set(preempted) == {"young"}
    assert len(scheduler.finished["old"].outputs) == 2 and len(scheduler.finished["young"].outputs) == 12


def test_random_pools_windows_and_chunks_always_make_progress():
    """Whatever the pool, the window and the portion size: every plan moves something, every
    request ends within a bounded number of steps with the tokens it produces in a roomy pool,
    and no page is lost on the way."""
    import random
    rng = random.Random(11)
    preemptions = 0
    for case in range(60):
        page_size = rng.choice([2, 4, 16])
        window = rng.choice([None, 24])
        chunk = rng.choice([1, 3, 8, 32])
        budget = rng.choice([chunk, 2 * chunk + 3, 64])
        n_requests = rng.randint(2, 6)
        prompts = {f"r{i}": [rng.randint(1, 40) for _ in range(rng.randint(1, 90))]
                   for i in range(n_requests)}
        num_predict = rng.randint(1, 12)
        longest = max(len(p) for p in prompts.values()) + num_predict
        pages_for_one = (longest + page_size - 1) // page_size
        if window is not None:
            pages_for_one = min(pages_for_one, (window - 1 + page_size - 1) // page_size + 2)
        pages = pages_for_one + rng.randint(0, pages_for_one)
        config = dict(page_size=page_size, window=window, max_num_seqs=rng.choice([2, 4]),
                      max_num_batched_tokens=budget, prefill_chunk=chunk, max_model_len=4096)
        expected = outputs_in_roomy_pool(prompts, num_predict, **config)
        cache, scheduler = make(pages=pages, **config)
        for name, prompt in prompts.items():
            scheduler.add(name, prompt, sampling(num_predict=num_predict, num_ctx=4096))
        total = sum(len(p) + num_predict for p in prompts.values())
        steps = 0
        while scheduler.has_work():
            plan, _ = run_step(cache, scheduler)
            assert plan.entries, (case, "empty plan")
            steps += 1
            assert steps <= 40 * total, (case, "no end in sight")
        for name in prompts:
            done = scheduler.finished[name]
            assert done.finish_reason == "length" and done.outputs == expected[name], (case, name)
        assert cache.free_pages() == [pages], case
        preemptions += scheduler.num_preemptions
    assert preemptions > 20             # the cases do run out of pages


def test_window_only_pool_too_small_is_refused_at_add_not_inside_a_step():
    cache, scheduler = make(pages=2, page_size=4, window=8)
    with pytest.raises(RequestRefused):
        scheduler.add("a", [1] * 30, sampling(num_predict=4))      # a window of 8 spans up to 4 pages
    scheduler.add("b", [1] * 5, sampling(num_predict=3))           # 8 tokens: 2 pages are enough
    run_all(cache, scheduler)
    assert len(scheduler.finished["b"].outputs) == 3


def test_trace_lines_are_checked_before_they_reach_the_engine():
    from matricxon_b200.engine.replay import TraceFormatError, parse_trace_line

    step, entries, end = parse_trace_line(
        '{"step": 3, "entries": [{"id": 7, "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["x", 9]}')
    assert step == 3 and entries == [{"id": "7", "tokens": [5, 17, 3], "want": [0, 2]}] and end == ["x", "9"]
    assert parse_trace_line('{"step": 0}') == (0, [], [])
    for line in ('{"step": 0', '[1, 2]', '{"entries": []}', '{"step": 0, "entries": {}}',
                 '{"step": 0, "entries": [{"id": "a"}]}', '{"step": 0, "entries": [{"id": "a", "tokens": []}]}',
                 '{"step": 0, "entries": [{"id": "a", "tokens": [1.5]}]}',
                 '{"step": 0, "entries": [{"id": "a", "tokens": [true]}]}',
                 '{"step": 0, "entries": [{"id": "a", "tokens": [1], "want": "all"}]}',
                 '{"step": 0, "entries": [], "end": "a"}'):
        with pytest.raises(TraceFormatError):
            parse_trace_line(line)

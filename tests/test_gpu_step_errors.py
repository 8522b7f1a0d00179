"""Faults of a step, made on the host (nothing here faults the GPU): entries the step function
refuses before it launches anything, and a token id that only the embedding kernel sees (it
writes zeros, sets a status bit, and the engine voids the step). The reference isolates a
failing reply from the others of its batch (app/runtime/batch_decode.py:82-83,101-105; tested
with a decoder that raises for one reply, tests/unit/test_batching_scheduler.py:126-149)."""

import pytest
import torch

from tiny_configs import TINY, random_ids, tiny_config, tiny_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_model(name="A", dtype="float32"):
    from matricxon_b200.engine.core import model_from_tensors

    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    return model_from_tensors(tiny_config(name), tiny_tensors(name, store), dtype=dtype, device=DEV)


def test_step_runner_refuses_malformed_entries_before_anything_is_reserved():
    from matricxon_b200.engine.core import EngineCore
    from matricxon_b200.engine.step import StepEntry, StepError

    model = make_model()
    vocab = TINY["A"][0]["vocab_size"]
    core = EngineCore(model, max_cache_tokens=128, max_requests=4)
    cache, runner = core.cache, core.runner
    for name in "ab":
        cache.add_request(name)
    free = cache.free_pages()
    cases = [
        ([StepEntry("a", [1, 2]), StepEntry("a", [3])], ["a"], "appears twice"),
        ([StepEntry("a", [1, 2]), StepEntry("ghost", [3])], ["ghost"], "not live"),
        ([StepEntry("a", [1, vocab]), StepEntry("b", [3])], ["a"], "outside the vocabulary"),
        ([StepEntry("a", [1, -1]), StepEntry("b", [3])], ["a"], "outside the vocabulary"),
        ([StepEntry("a", [1, 2], [2]), StepEntry("b", [3], [0])], ["a"], "wants logits at 2"),
        ([StepEntry("a", []), StepEntry("b", [vocab + 7])], ["a", "b"], "brings no tokens"),
    ]
    for entries, at_fault, text in cases:
        with pytest.raises(StepError) as caught:
            runner.run(entries)
        assert caught.value.request_ids == at_fault and text in str(caught.value)
        assert cache.free_pages() == free and cache.record("a").length == 0 and cache.record("a").reserved == 0
        cache.check_invariants()
    with pytest.raises(StepError):
        runner.run([])
    # the runner is as good as new: the same requests run
    logits = runner.run([StepEntry("a", [1, 2], [1]), StepEntry("b", [3], [0])])
    runner.check_status()
    assert logits.shape == (2, vocab) and bool(torch.isfinite(logits).all())


def test_a_bad_id_seen_by_the_host_ends_its_request_and_the_others_go_on():
    from matricxon_b200 import ChatEngine, SamplingConfig

    model = make_model()
    vocab = TINY["A"][0]["vocab_size"]
    sampling = SamplingConfig(temperature=0.0, num_predict=6, num_ctx=64)
    prompts = {name: random_ids(n, vocab, seed=n) for name, n in (("good1", 9), ("bad", 12), ("good2", 20))}
    alone = {}
    for name in ("good1", "good2"):
        engine = ChatEngine(model, max_cache_tokens=256, max_active=4, prefill_chunk=8, max_model_len=128)
        rid = engine.add_request(prompts[name], sampling)
        while engine.has_unfinished():
            engine.step()
        alone[name] = engine.result(rid).token_ids
    engine = ChatEngine(model, max_cache_tokens=256, max_active=4, prefill_chunk=8, max_model_len=128)
    from matricxon_b200.engine.scheduler import RequestRefused
    with pytest.raises(RequestRefused):
        engine.add_request([1, vocab, 2], sampling)                # caught at the door
    for name, prompt in prompts.items():
        engine.add_request(prompt, sampling, request_id=name)
    with pytest.raises(RequestRefused):
        engine.add_request([1, 2], sampling, request_id="bad")      # an id in use
    # the id goes wrong after admission, in the second portion of the prompt
    next(s for s in engine.scheduler.waiting if s.request_id == "bad").prompt[10] = vocab + 5
    events = []
    for _ in range(200):
        if not engine.has_unfinished():
            break
        events.extend(engine.step())
    assert not engine.has_unfinished()
    assert ("bad", None, True) in events
    failed = engine.result("bad")
    assert failed.finish_reason == "error" and "outside the vocabulary" in failed.error and failed.token_ids == []
    for name in ("good1", "good2"):
        result = engine.result(name)
        assert result.finish_reason == "length" and result.token_ids == alone[name]
    assert engine.core.cache.free_pages() == [16]
    engine.core.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_bad_id_seen_only_by_the_kernel_voids_the_step_for_its_requests(dtype):
    """With the host's scan switched off the embedding kernel is the one that notices: it
    writes zeros for the row and sets a status bit. The requests of that step end with
    ``error``; a request admitted later runs as if nothing had happened."""
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig

    model = make_model("B", dtype)
    vocab = TINY["B"][0]["vocab_size"]
    sampling = SamplingConfig(temperature=0.0, num_predict=5, num_ctx=128)
    later_prompt = random_ids(11, vocab, seed=3)
    expected = ChatEngine(model, max_cache_tokens=256, max_active=4, max_model_len=256).generate(
        GenerationRequest(later_prompt, sampling)).token_ids
    engine = ChatEngine(model, max_cache_tokens=256, max_active=4, max_model_len=256)
    engine.core.runner.check_ids_on_host = False
    engine.add_request(random_ids(7, vocab, seed=1), sampling, request_id="neighbour")
    engine.add_request(random_ids(9, vocab, seed=2), sampling, request_id="bad")
    engine.scheduler.waiting[1].prompt[4] = vocab + 1
    events = engine.step()
    assert sorted(events) == [("bad", None, True), ("neighbour", None, True)]
    for name in ("bad", "neighbour"):
        result = engine.result(name)
        assert result.finish_reason == "error" and "outside the vocabulary" in result.error
    assert not engine.has_unfinished() and engine.core.cache.free_pages() == [16]
    engine.core.runner.check_ids_on_host = True
    assert engine.generate(GenerationRequest(later_prompt, sampling)).token_ids == expected


def test_a_bad_id_fed_from_the_device_is_reported_by_the_status_word():
    """A decode step that takes its ids from the device (the step queued ahead) is the one case
    the host cannot scan."""
    from matricxon_b200.engine.core import EngineCore
    from matricxon_b200.engine.step import StepEntry, StepError

    model = make_model("A", "bfloat16")
    vocab = TINY["A"][0]["vocab_size"]
    core = EngineCore(model, max_cache_tokens=128, max_requests=4)
    cache, runner = core.cache, core.runner
    for name in "ab":
        cache.add_request(name)
    runner.run([StepEntry("a", [1, 2, 3]), StepEntry("b", [4, 5])])
    runner.run([StepEntry("a", [6], [0]), StepEntry("b", [7], [0])])        # captures the two-row graph
    runner.check_status()
    feed = torch.tensor([8, vocab + 9], dtype=torch.int32, device=DEV)
    assert runner.can_feed_from_device([StepEntry("a", [0], [0]), StepEntry("b", [0], [0])])
    runner.run([StepEntry("a", [0], [0]), StepEntry("b", [0], [0])], token_feed=feed)
    with pytest.raises(StepError) as caught:
        runner.check_status()
    assert "outside the vocabulary" in str(caught.value) and caught.value.request_ids == []
    runner.check_status()                                           # the word was cleared

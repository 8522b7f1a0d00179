"""Generation through the Python entry point and the sampling kernel against the plain sampler."""

import numpy as np
import pytest
import torch

from plain_reference import plain_config, plain_forward, plain_sample
from tiny_configs import TINY, random_ids, tiny_config, tiny_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build(name, dtype):
    from matricxon_b200.engine.core import model_from_tensors

    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = tiny_tensors(name, store)
    model = model_from_tensors(tiny_config(name), tensors, dtype=dtype, device=DEV)
    return model, plain_config(TINY[name][0]), {k: v.float() for k, v in tensors.items()}


# ------------------------------------------------------------------ the sampling kernel alone
def sample_rows(logits, configs, generated=None, uniforms=None):
    from matricxon_b200.sampling.sampler import BatchSampler, RequestSampler

    samplers = []
    for i, config in enumerate(configs):
        s = RequestSampler(config)
        for token in (generated[i] if generated else []):
            s.accept(token)
        if uniforms is not None:
            s.next_uniform = (lambda u: (lambda ahead=0: u))(uniforms[i])
        samplers.append(s)
    batch = BatchSampler(DEV, logits.shape[1])
    return batch.sample(logits.to(DEV), samplers), samplers


def test_greedy_takes_the_first_of_equal_maxima_and_ignores_other_options():
    from matricxon_b200 import SamplingConfig

    logits = torch.randn(5, 1000)
    logits[0, [17, 400, 999]] = 9.0
    logits[1, 999] = 50.0
    logits[2, 0] = 50.0
    tokens, _ = sample_rows(logits, [SamplingConfig(temperature=0.0, seed=1)] * 5)
    assert tokens[:3] == [17, 999, 0]
    assert tokens == [int(torch.argmax(row)) for row in logits]
    tokens, _ = sample_rows(logits, [SamplingConfig(temperature=-1.0, top_k=1, top_p=0.1, repeat_penalty=1.0)] * 5)
    assert tokens == [int(torch.argmax(row)) for row in logits]


@pytest.mark.parametrize("vocab", [1000, 49152, 300000])
def test_greedy_with_a_repeat_penalty_judges_penalised_ids_by_their_adjusted_scores(vocab):
    """Greedy rows take a path of their own (one pass, penalised ids marked in a bitmap; vocabularies
    whose bitmap does not fit keep the general path): the best id is penalised below the second, a
    negative best score gets more negative, an id that is generated and still pending on the device is
    penalised once, a penalty below one can lift a generated id to the top."""
    from matricxon_b200 import SamplingConfig
    from matricxon_b200.sampling.sampler import BatchSampler, RequestSampler

    torch.manual_seed(vocab)
    logits = torch.randn(6, vocab)
    logits[0, 7], logits[0, 900] = 10.0, 9.5          # 7 is generated: 10 / 1.5 < 9.5
    logits[1] = -torch.rand(vocab) - 1.0
    logits[1, 33], logits[1, 34] = -0.5, -0.6         # 33 is generated: -0.5 * 1.5 < -0.6
    logits[2, 5], logits[2, 6] = 10.0, 9.0            # 5 is pending only: penalised
    logits[3, 5], logits[3, 6] = 10.0, 7.0            # 5 is generated and pending: once (10 / 1.3 > 7), not twice (10 / 1.69 < 7)
    logits[4, 8], logits[4, 9] = 4.0, 5.0             # penalty 0.5 lifts the generated 8 above 9
    configs = [SamplingConfig(temperature=0.0, repeat_penalty=p) for p in (1.5, 1.5, 1.5, 1.3, 0.5, 1.0)]
    generated = [[7, 1, 2], [33], [], [5], [8], [int(torch.argmax(logits[5]))]]
    pending = [-1, -1, 5, 5, -1, -1]
    samplers = []
    for config, ids in zip(configs, generated):
        sampler = RequestSampler(config)
        for token in ids:
            sampler.accept(token)
        samplers.append(sampler)
    batch = BatchSampler(DEV, vocab)
    feed = torch.tensor(pending, dtype=torch.int32, device=DEV)
    tokens = batch.read(batch.launch(logits.to(DEV), samplers, pending=feed))
    expected = []
    for row, config, ids, extra in zip(logits, configs, generated, pending):
        seen = ids + ([extra] if extra >= 0 else [])
        expected.append(plain_sample(row, seen, 0.0, 0, 1.0, config.repeat_penalty, 0.5))
    assert tokens == expected
    assert tokens[:5] == [900, 34, 6, 5, 8] and tokens[5] == int(torch.argmax(logits[5]))


@pytest.mark.parametrize("top_k,top_p,penalty,temperature", [
    (0, 1.0, 1.0, 1.0), (40, 0.9, 1.1, 0.8), (5, 1.0, 1.0, 0.7), (0, 0.6, 1.0, 1.3), (3, 0.5, 1.5, 0.5)])
def test_sampling_matches_plain_sampler_over_a_quantile_sweep(top_k, top_p, penalty, temperature):
    """Sweeps u over quantiles, as the reference tests its fused sampler
    (tests/unit/test_fused_ops.py:116-128): the kernel and the plain sampler must pick the
    same token except where u falls on a boundary within rounding."""
    from matricxon_b200 import SamplingConfig

    vocab, n = 1000, 600
    torch.manual_seed(top_k + int(top_p * 10))
    row = torch.randn(vocab) * 2.0
    generated = [3, 17, 17, 999, int(torch.argmax(row))]
    config = SamplingConfig(temperature=temperature, top_k=top_k, top_p=top_p, repeat_penalty=penalty, seed=0)
    uniforms = [(i + 0.5) / n for i in range(n)]
    logits = row.repeat(n, 1)
    tokens, _ = sample_rows(logits, [config] * n, [generated] * n, uniforms)
    expected = [plain_sample(row, generated, temperature, top_k, top_p, penalty, u) for u in uniforms]
    mismatches = sum(a != b for a, b in zip(tokens, expected))
    assert mismatches <= 1, mismatches
    if top_k:
        assert len(set(tokens)) <= top_k


def test_top_k_keeps_ties_and_vocab_not_a_multiple_of_anything():
    from matricxon_b200 import SamplingConfig

    vocab = 1237
    row = torch.full((vocab,), -5.0)
    row[[10, 20, 30]] = 2.0                       # three-way tie at the top, k = 2 keeps all three
    n = 300
    uniforms = [(i + 0.5) / n for i in range(n)]
    tokens, _ = sample_rows(row.repeat(n, 1), [SamplingConfig(temperature=1.0, top_k=2, top_p=1.0,
                                                               repeat_penalty=1.0)] * n, None, uniforms)
    counts = {t: tokens.count(t) for t in set(tokens)}
    assert set(counts) == {10, 20, 30} and all(abs(c - 100) <= 1 for c in counts.values())
    # u close to 1 lands on the last candidate, never outside the vocabulary
    tokens, _ = sample_rows(row.repeat(2, 1), [SamplingConfig(temperature=1.0, top_k=0, top_p=1.0,
                                                               repeat_penalty=1.0)] * 2, None, [0.9999999, 0.0])
    assert 0 <= tokens[0] < vocab and tokens[1] == 0


def test_rows_are_sampled_independently_with_their_own_options():
    from matricxon_b200 import SamplingConfig

    torch.manual_seed(5)
    logits = torch.randn(4, 512)
    configs = [SamplingConfig(temperature=0.0), SamplingConfig(temperature=0.7, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=3),
               SamplingConfig(temperature=1.0, top_k=4, top_p=0.8, repeat_penalty=1.3, seed=4), SamplingConfig(temperature=0.0)]
    generated = [[], [1, 2], [int(torch.argmax(logits[2]))], []]
    together, samplers = sample_rows(logits, configs, generated)
    for i in range(4):
        alone, _ = sample_rows(logits[i:i + 1], [configs[i]], [generated[i]])
        assert alone[0] == together[i]
        expected = plain_sample(logits[i], generated[i], configs[i].temperature, configs[i].top_k,
                                configs[i].top_p, configs[i].repeat_penalty, samplers[i].next_uniform())
        assert together[i] == expected


# ------------------------------------------------------------------ the entry point
def plain_greedy_check(cfg, weights, prompt, outputs, dtype):
    """Every generated token must be the plain implementation's argmax given what came before
    (in bfloat16: within the rounding of the logits)."""
    logits = plain_forward(cfg, weights, prompt + outputs).numpy()
    for i, token in enumerate(outputs):
        row = logits[len(prompt) + i - 1]
        slack = 0.0 if dtype == "float32" else 0.03 * np.abs(row).max()
        assert row[token] >= row.max() - slack - 1e-6, (i, token, int(row.argmax()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_config_a(dtype):
    """Tiny A: prompts of 5, 17, 40 and 64 tokens (two cross the window), 16 greedy steps each,
    alone and all four together."""
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig

    model, cfg, weights = build("A", dtype)
    engine = ChatEngine(model, max_cache_tokens=512, max_active=4, max_batched_tokens=64, prefill_chunk=7,
                        max_model_len=128)
    prompts = [random_ids(n, cfg["vocab"], seed=n) for n in (5, 17, 40, 64)]
    sampling = SamplingConfig(temperature=0.0, repeat_penalty=1.0, num_predict=16, num_ctx=128, seed=0)
    alone = [engine.generate(GenerationRequest(p, sampling)) for p in prompts]
    for prompt, result in zip(prompts, alone):
        assert len(result.token_ids) == 16 and result.finish_reason == "length"
        plain_greedy_check(cfg, weights, prompt, result.token_ids, dtype)
    together = engine.generate_batch([GenerationRequest(p, sampling) for p in prompts])
    if dtype == "float32":
        assert [r.token_ids for r in together] == [r.token_ids for r in alone]
    for prompt, result in zip(prompts, together):
        plain_greedy_check(cfg, weights, prompt, result.token_ids, dtype)
    assert engine.core.cache.free_pages() == [32]
    streamed = list(engine.stream(GenerationRequest(prompts[1], sampling)))
    assert dtype != "float32" or streamed == alone[1].token_ids


def test_seeded_temperature_generation_config_b():
    """Tiny B: prompts of 1, 3, 23, 24, 25 and 100 tokens, 32 steps at temperature 0.7 with a
    seed; portions of 10 prompt tokens run beside decoding requests. The tokens equal the
    plain sampler's on the plain logits with the same uniforms, alone and batched."""
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig
    from matricxon_b200.sampling.sampler import uniform_for

    model, cfg, weights = build("B", "float32")
    engine = ChatEngine(model, max_cache_tokens=6 * 192, max_active=6, max_batched_tokens=24,
                        prefill_chunk=10, max_model_len=256)
    prompts = [random_ids(n, cfg["vocab"], seed=50 + n) for n in (1, 3, 23, 24, 25, 100)]
    configs = [SamplingConfig(temperature=0.7, top_k=0, top_p=1.0, repeat_penalty=1.0, num_predict=32,
                              num_ctx=256, seed=100 + i) for i in range(len(prompts))]
    batched = engine.generate_batch([GenerationRequest(p, c) for p, c in zip(prompts, configs)])
    assert engine.steps < sum(32 + len(p) // 10 + 1 for p in prompts)       # steps were shared
    for i, (prompt, result) in enumerate(zip(prompts, batched)):
        assert len(result.token_ids) == 32
        logits = plain_forward(cfg, weights, prompt + result.token_ids)
        for step, token in enumerate(result.token_ids):
            row = logits[len(prompt) + step - 1].float()
            expected = plain_sample(row, result.token_ids[:step], 0.7, 0, 1.0, 1.0, uniform_for(100 + i, step))
            assert token == expected, (i, step)
    alone = engine.generate(GenerationRequest(prompts[3], configs[3]))
    assert alone.token_ids == batched[3].token_ids
    other_seed = engine.generate(GenerationRequest(prompts[3], SamplingConfig(
        temperature=0.7, top_k=0, top_p=1.0, repeat_penalty=1.0, num_predict=32, num_ctx=256, seed=7)))
    assert other_seed.token_ids != alone.token_ids


def test_preemption_in_the_engine_leaves_tokens_unchanged():
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig

    model, cfg, weights = build("B", "float32")
    prompts = [random_ids(n, cfg["vocab"], seed=70 + n) for n in (30, 28, 26)]
    configs = [SamplingConfig(temperature=0.9, top_k=20, top_p=0.95, repeat_penalty=1.1, num_predict=40,
                              num_ctx=256, seed=i) for i in range(3)]
    roomy = ChatEngine(model, max_cache_tokens=1024, max_active=4, max_model_len=256)
    expected = roomy.generate_batch([GenerationRequest(p, c) for p, c in zip(prompts, configs)])
    # each request holds 2 to 3 pages of 16 while it runs (window 24): 5 pages cannot serve three
    tight = ChatEngine(model, max_cache_tokens=5 * 16, max_active=4, max_model_len=256)
    got = tight.generate_batch([GenerationRequest(p, c) for p, c in zip(prompts, configs)])
    assert tight.scheduler.num_preemptions >= 1
    assert [r.token_ids for r in got] == [r.token_ids for r in expected]
    assert tight.core.cache.free_pages() == [5]


def test_eos_and_cancel():
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig

    model, cfg, _ = build("A", "float32")
    prompt = random_ids(9, cfg["vocab"], 1)
    sampling = SamplingConfig(temperature=0.0, num_predict=12, num_ctx=64)
    free_run = ChatEngine(model, max_cache_tokens=256, max_active=2, max_model_len=128).generate(
        GenerationRequest(prompt, sampling))
    eos = free_run.token_ids[4]
    first = free_run.token_ids.index(eos)
    engine = ChatEngine(model, eos_token_ids={eos}, max_cache_tokens=256, max_active=2, max_model_len=128)
    stopped = engine.generate(GenerationRequest(prompt, sampling))
    assert stopped.finish_reason == "stop" and stopped.token_ids == free_run.token_ids[:first + 1]
    engine = ChatEngine(model, max_cache_tokens=256, max_active=2, max_model_len=128)
    rid = engine.add_request(prompt, sampling)
    engine.step()
    assert engine.cancel(rid) and engine.result(rid).finish_reason == "cancelled"
    assert not engine.has_unfinished() and engine.core.cache.free_pages() == [16]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_queued_ahead_change_no_token(dtype):
    """While everybody decodes, the engine queues the next step before it has read the ids of
    the running one (they are fed on the device, and the repeat penalty counts them there). The
    tokens must equal those of deciding step by step: with a repeat penalty, seeded
    temperature sampling and different lengths; in 32-bit (where another batch around a request
    cannot move a token) also with a stop token in the middle of one request, a request that
    arrives while others decode, and one that is cancelled."""
    from matricxon_b200 import ChatEngine, SamplingConfig

    model, cfg, _ = build("B", dtype)
    eventful = dtype == "float32"
    prompts = [random_ids(n, cfg["vocab"], seed=90 + n) for n in (5, 17, 33, 12)]
    configs = [
        SamplingConfig(temperature=0.0, repeat_penalty=1.6, num_predict=40, num_ctx=256),
        SamplingConfig(temperature=0.9, top_k=30, top_p=0.9, repeat_penalty=1.3, num_predict=25, num_ctx=256, seed=3),
        SamplingConfig(temperature=1.2, top_k=0, top_p=1.0, repeat_penalty=1.0, num_predict=48, num_ctx=256, seed=4),
        SamplingConfig(temperature=0.5, top_k=8, top_p=1.0, repeat_penalty=1.2, num_predict=30, num_ctx=256, seed=5),
    ]

    def run(look_ahead, eos=()):
        engine = ChatEngine(model, eos_token_ids=eos, max_cache_tokens=1024, max_active=4, max_model_len=256,
                            look_ahead=look_ahead)
        ids = [engine.add_request(p, c) for p, c in zip(prompts[:3], configs[:3])]
        if not eventful:
            ids.append(engine.add_request(prompts[3], configs[3]))
        while engine.has_unfinished():
            engine.step()
            if eventful and engine.steps == 9:
                ids.append(engine.add_request(prompts[3], configs[3]))
            if eventful and engine.steps == 20:
                engine.cancel(ids[2])
        assert engine.core.cache.free_pages() == [p.num_pages for p in engine.core.cache.pools]
        results = [engine.result(i) for i in ids]
        return engine, [(r.token_ids, r.finish_reason) for r in results]

    plain, expected = run(False)
    assert plain.steps_ahead == 0
    ahead, got = run(True)
    assert ahead.steps_ahead >= 20 and got == expected
    assert len(set(expected[0][0])) > 8                       # the penalty did shape the greedy request
    if eventful:
        assert expected[2][1] == "cancelled" and len(expected[2][0]) < 48
        # a stop token that the first request meets in mid-flight: its row of the step ahead is dropped
        stop = expected[0][0][15]
        _, expected_stop = run(False, eos={stop})
        ahead, got_stop = run(True, eos={stop})
        assert got_stop == expected_stop and ahead.steps_ahead >= 10
        assert got_stop[0][1] == "stop" and len(got_stop[0][0]) <= 16


def test_command_line(tmp_path):
    import subprocess
    import sys

    from tiny_configs import write_tiny_model
    from trace_utils import ROOT

    folder = write_tiny_model(tmp_path / "m", "A")
    out = subprocess.run([sys.executable, "-m", "matricxon_b200.generate", "--model-dir", str(folder),
                          "--prompt-ids", "5,17,3", "--num-predict", "6", "--dtype", "float32"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    assert "finish_reason:  length" in out.stdout and "architecture: Starcoder2ForCausalLM" in out.stdout
    ids_line = [l for l in out.stdout.splitlines() if l.startswith("generated ids:")][0]
    assert len(eval(ids_line.split(":", 1)[1])) == 6

"""Real StarCoder2 layer sizes, two layers, random weights: the engine against the plain
implementation under every way of cutting the work, in float32 and in bfloat16.

  3B sizes: hidden 3072, 24 heads, 2 KV heads (groups of 12), intermediate 12288, tied head;
  7B sizes: hidden 4608, 36 heads, 4 KV heads (groups of 9), intermediate 18432, untied head.

A window of 96 makes the sliding window bite inside a 200-token request; the configurations' own
window of 4096 is run as well (7B sizes), and by the long-context test below. This is where the
tcgen05 products (steps of more than 128 rows), the library product with the engine's epilogue
(17 to 128 rows), the 16-row product and all three attention kernels meet inside the engine."""

import numpy as np
import pytest
import torch

from plain_reference import (
    plain_config,
    plain_embedding,
    plain_forward,
    plain_layer,
    plain_layernorm,
)

pytestmark = pytest.mark.gpu

COMMON = {
    "model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"], "num_hidden_layers": 2,
    "head_dim": 128, "vocab_size": 49152, "max_position_embeddings": 16384, "norm_epsilon": 1e-5,
    "use_bias": True, "hidden_act": "gelu_pytorch_tanh",
}
SIZES_3B = dict(COMMON, hidden_size=3072, num_attention_heads=24, num_key_value_heads=2,
                intermediate_size=12288, rope_theta=999999.4420358813, tie_word_embeddings=True)
SIZES_7B = dict(COMMON, hidden_size=4608, num_attention_heads=36, num_key_value_heads=4,
                intermediate_size=18432, rope_theta=1000000.0, tie_word_embeddings=False)
GEOMETRIES = {"3b-window96": dict(SIZES_3B, sliding_window=96), "7b-window96": dict(SIZES_7B, sliding_window=96),
              "7b-window4096": dict(SIZES_7B, sliding_window=4096)}
LENGTHS = {"a": 200, "b": 77, "c": 130}
_MEMO: dict = {}        # what two parametrisations of one test share (weights, the plain logits)


def make_material(raw, seed=3):
    from matricxon_b200.config.registry import config_from_dict
    from matricxon_b200.weights.random_init import RandomInit, random_tensors

    config = config_from_dict(dict(raw))
    tensors = random_tensors(config, seed=seed, init=RandomInit(0.02, 0.02, 0.0, 0.0), store_dtype=torch.bfloat16)
    return config, tensors, plain_config(raw), {k: v.float() for k, v in tensors.items()}


@pytest.fixture(scope="module", params=list(GEOMETRIES))
def material(request):
    raw = GEOMETRIES[request.param]
    config, tensors, cfg, weights = make_material(raw)
    generator = torch.Generator().manual_seed(9)
    prompts = {rid: torch.randint(0, raw["vocab_size"], (n,), generator=generator).tolist()
               for rid, n in LENGTHS.items()}
    reference = {rid: plain_forward(cfg, weights, ids, dtype=torch.float32).numpy() for rid, ids in prompts.items()}
    del weights
    return config, tensors, prompts, reference


def run_trace(replayer, steps):
    """steps: list of (portions, ended); portions: list of (request, tokens). Every position is wanted."""
    logits, progress = {}, {}
    for portions, ended in steps:
        entries, keys = [], []
        for rid, tokens in portions:
            start = progress.get(rid, 0)
            entries.append({"id": rid, "tokens": tokens, "want": list(range(len(tokens)))})
            keys.extend((rid, start + i) for i in range(len(tokens)))
            progress[rid] = start + len(tokens)
        out = replayer.step(entries, ended)
        for key, row in zip(keys, out.numpy()):
            logits[key] = row
    return logits


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_every_cutting(material, dtype):
    from matricxon_b200.engine.core import model_from_tensors
    from matricxon_b200.engine.replay import TraceReplayer

    config, tensors, prompts, reference = material
    model = model_from_tensors(config, tensors, dtype=dtype, device="cuda:0")
    replayer = TraceReplayer(None, dtype, max_tokens=512, model=model, poison_cache=True)

    def compare(logits, rid, tag):
        ref = reference[rid]
        got = np.stack([logits[(rid, i)] for i in range(len(ref))])
        worst = np.abs(got - ref).max(axis=1)
        limit = (2e-4 if dtype == "float32" else 0.03) * float(np.abs(ref).max())
        bad = np.nonzero(worst > limit)[0]
        assert bad.size == 0, f"{tag} {rid}: first wrong position {bad[0]}, error {worst[bad[0]]:.3e} > {limit:.2e}"

    # whole
    for rid, ids in prompts.items():
        compare(run_trace(replayer, [([(rid, ids)], [rid])]), rid, "whole")
    # most in one step, the last 32 one by one
    ids = prompts["a"]
    steps = [([("a", ids[:-32])], [])] + [([("a", [t])], []) for t in ids[-32:-1]] + [([("a", ids[-1:])], ["a"])]
    compare(run_trace(replayer, steps), "a", "tail")
    # portions of changing size, down to two tokens
    sizes, steps, start = [64, 2, 33, 7, 2, 50, 16, 26], [], 0
    for size in sizes:
        steps.append(([("a", ids[start:start + size])], ["a"] if start + size == len(ids) else []))
        start += size
    assert start == len(ids)
    compare(run_trace(replayer, steps), "a", "portions")
    # mixed: portions of one request beside decoded tokens of others, pages used again
    done = {rid: 0 for rid in prompts}
    plan = {"a": [100, 60, 38, 1, 1], "b": [70, 1, 1, 1, 1, 1, 1, 1], "c": [2, 90, 30, 4, 1, 1, 1, 1]}
    steps = []
    for turn in range(8):
        portions, ended = [], []
        for rid, cuts in plan.items():
            if turn < len(cuts):
                n = cuts[turn]
                portions.append((rid, prompts[rid][done[rid]:done[rid] + n]))
                done[rid] += n
                if done[rid] == len(prompts[rid]):
                    ended.append(rid)
        steps.append((portions, ended))
    assert all(done[rid] == len(prompts[rid]) for rid in prompts)
    logits = run_trace(replayer, steps)
    for rid in prompts:
        compare(logits, rid, "mixed")
    assert replayer.core.cache.pages_reused > 0
    assert replayer.core.cache.free_pages() == [32]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_short_portion_after_three_thousand_cached_tokens(dtype):
    """3B sizes with the configuration's own window of 4096: 3,036 tokens in one step, then a
    64-token portion (few tiles over a long context: the tcgen05 attention shares each tile's keys
    out between blocks), two decoded tokens (the narrow kernel with split keys) and a 17-token
    portion (library product rows beside tcgen05 attention tiles)."""
    from matricxon_b200.engine.core import model_from_tensors
    from matricxon_b200.engine.replay import TraceReplayer

    total, cuts = 3119, [3036, 64, 1, 1, 17]
    assert sum(cuts) == total
    if "long" not in _MEMO:
        config, tensors, cfg, weights = make_material(dict(SIZES_3B, sliding_window=4096), seed=4)
        ids = torch.randint(0, config.vocab_size, (total,), generator=torch.Generator().manual_seed(2)).tolist()
        _MEMO["long"] = (config, tensors, ids, plain_forward(cfg, weights, ids, dtype=torch.float32)[cuts[0]:].numpy())
        del weights
    config, tensors, ids, reference = _MEMO["long"]
    model = model_from_tensors(config, tensors, dtype=dtype, device="cuda:0")
    replayer = TraceReplayer(None, dtype, max_tokens=3200, model=model, poison_cache=True)
    got, start = [], 0
    for index, size in enumerate(cuts):
        want = [] if index == 0 else list(range(size))
        out = replayer.step([{"id": "long", "tokens": ids[start:start + size], "want": want}],
                            ["long"] if start + size == total else [])
        if want:
            got.append(out.numpy())
        start += size
    got = np.concatenate(got)
    worst = np.abs(got - reference).max(axis=1)
    limit = (2e-4 if dtype == "float32" else 0.03) * float(np.abs(reference).max())
    bad = np.nonzero(worst > limit)[0]
    assert bad.size == 0, f"first wrong position {cuts[0] + bad[0]}, error {worst[bad[0]]:.3e} > {limit:.2e}"


def test_block_tables_longer_than_a_thousand_pages():
    """A request of 17,000 tokens with a window of 4,096 and pages of 16: its block table has
    1,063 entries, of which about 257 still name a page (the tcgen05 attention keeps 1,024 entries
    in shared memory and reads the rest from global memory). One layer with heads of 128, so that
    the plain implementation can be asked for the last positions alone: with one layer, keys and
    values of a position depend on its own token only, and a query sees nothing older than its
    window, so the plain layer over the last 4,300 tokens at their true positions gives the same
    last 150 rows as it would over all 17,000."""
    from matricxon_b200.config.registry import config_from_dict
    from matricxon_b200.engine.core import model_from_tensors
    from matricxon_b200.engine.replay import TraceReplayer
    from matricxon_b200.weights.random_init import RandomInit, random_tensors

    raw = dict(COMMON, num_hidden_layers=1, hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
               intermediate_size=1024, vocab_size=1000, rope_theta=100000.0, sliding_window=4096,
               max_position_embeddings=32768, tie_word_embeddings=True)
    config = config_from_dict(raw)
    tensors = random_tensors(config, seed=6, init=RandomInit(0.05, 0.02, 0.0, 0.0), store_dtype=torch.bfloat16)
    cfg, weights = plain_config(raw), {k: v.float() for k, v in tensors.items()}
    total, tail, checked = 17000, 4300, 150
    ids = torch.randint(0, 1000, (total,), generator=torch.Generator().manual_seed(8)).tolist()
    x = plain_embedding(torch.tensor(ids[-tail:]), weights["model.embed_tokens.weight"])
    x = plain_layer(x, weights, 0, cfg, torch.arange(total - tail, total))
    x = plain_layernorm(x, weights["model.norm.weight"], weights["model.norm.bias"], cfg["eps"])
    reference = (x @ weights["model.embed_tokens.weight"].T)[-checked:].numpy()

    model = model_from_tensors(config, tensors, dtype="bfloat16", device="cuda:0")
    replayer = TraceReplayer(None, "bfloat16", max_tokens=12288, model=model, poison_cache=True)
    cuts = [4096] * 4 + [466, 100, 1, 1, 48]            # the last three steps hold the checked rows
    assert sum(cuts) == total and sum(cuts[-4:]) == checked
    got, start = [], 0
    for index, size in enumerate(cuts):
        want = list(range(size)) if index >= len(cuts) - 4 else []
        out = replayer.step([{"id": "long", "tokens": ids[start:start + size], "want": want}], [])
        if want:
            got.append(out.numpy())
        start += size
    record = replayer.core.cache.record("long")
    assert len(record.tables[0]) == (total + 15) // 16 == 1063
    assert 256 <= sum(page >= 0 for page in record.tables[0]) <= 258
    got = np.concatenate(got)
    worst = np.abs(got - reference).max(axis=1)
    limit = 0.03 * float(np.abs(reference).max())
    bad = np.nonzero(worst > limit)[0]
    assert bad.size == 0, f"first wrong position {total - checked + bad[0]}, error {worst[bad[0]]:.3e} > {limit:.2e}"


def test_preemption_and_a_stop_token_at_3b_layer_sizes():
    """The scheduler above the tcgen05 products and attention: a pool too small for three requests
    (somebody is preempted and recomputed as prompt + tokens, which moves its rows from the 16-row
    decode kernels to the prompt kernels), and a stop token. bfloat16 rounds differently on the two
    paths, so every token is checked against the plain implementation's logits given what came
    before it, not against the other run: the engine's logits lie within t = 3 % of the largest
    |logit| of the plain ones (what the logits tests above assert), so the token it takes as the
    largest is within 2 t of the plain maximum."""
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig
    from matricxon_b200.engine.core import model_from_tensors

    config, tensors, cfg, weights = make_material(dict(SIZES_3B, sliding_window=96), seed=5)
    model = model_from_tensors(config, tensors, dtype="bfloat16", device="cuda:0")
    generator = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in (150, 140, 33)]
    # no repeat penalty: with one, "greedy" is the largest penalised logit (app/runtime/sampler.py:108-117)
    sampling = SamplingConfig(temperature=0.0, repeat_penalty=1.0, num_predict=24, num_ctx=512)
    # each request holds up to 7 pages of 16 inside its window of 96; 14 pages cannot serve three
    tight = ChatEngine(model, max_cache_tokens=14 * 16, max_active=4, prefill_chunk=48, max_model_len=512)
    results = tight.generate_batch([GenerationRequest(p, sampling) for p in prompts])
    assert tight.scheduler.num_preemptions >= 1
    assert tight.core.cache.free_pages() == [14]
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 24 and result.finish_reason == "length"
        logits = plain_forward(cfg, weights, prompt + result.token_ids, dtype=torch.float32).numpy()
        for i, token in enumerate(result.token_ids):
            row = logits[len(prompt) + i - 1]
            assert row[token] >= row.max() - 2 * 0.03 * np.abs(row).max(), (i, token, int(row.argmax()))
    # a stop token: the same engine, the same request alone, stops where that token first appears
    free_run = results[2].token_ids
    alone = ChatEngine(model, max_cache_tokens=512, max_active=2, prefill_chunk=48, max_model_len=512)
    again = alone.generate(GenerationRequest(prompts[2], sampling)).token_ids
    eos = again[6]
    stopping = ChatEngine(model, eos_token_ids={eos}, max_cache_tokens=512, max_active=2, prefill_chunk=48,
                          max_model_len=512)
    stopped = stopping.generate(GenerationRequest(prompts[2], sampling))
    assert stopped.finish_reason == "stop" and stopped.token_ids == again[:again.index(eos) + 1]
    assert len(free_run) == 24

"""Decode steps of many rows: 24 and 64 requests decoding together through the captured graphs of
32 and 64 rows (where the products leave the 16-row kernel for the library product with the
engine's epilogue, and the attention runs 64 narrow tiles), and 70 requests in one eager step
beyond the largest captured size. Logits of every decoded position against the plain
implementation, in float32 and in bfloat16, for tiny B and for two layers of StarCoder2-3B sizes.
The reference batches up to 64 replies' decode steps the same way
(app/runtime/batch_decode.py:63-87; tests/unit/test_batched_decode.py:46-120)."""

import numpy as np
import pytest
import torch

from plain_reference import plain_config, plain_forward
from tiny_configs import TINY, tiny_config, tiny_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DECODE_STEPS = 20

RAW_3B_TWO_LAYERS = {
    "model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 3072, "num_attention_heads": 24, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 49152, "rope_theta": 999999.4420358813,
    "sliding_window": 96, "max_position_embeddings": 16384, "norm_epsilon": 1e-5, "use_bias": True,
    "tie_word_embeddings": True, "hidden_act": "gelu_pytorch_tanh",
}


def material(kind, dtype):
    from matricxon_b200.config.registry import config_from_dict
    from matricxon_b200.engine.core import model_from_tensors
    from matricxon_b200.weights.random_init import RandomInit, random_tensors

    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    if kind == "B":
        raw, config, tensors = TINY["B"][0], tiny_config("B"), tiny_tensors("B", store)
    else:
        raw = RAW_3B_TWO_LAYERS
        config = config_from_dict(dict(raw))
        tensors = random_tensors(config, seed=3, init=RandomInit(0.02, 0.02, 0.0, 0.0), store_dtype=torch.bfloat16)
    model = model_from_tensors(config, tensors, dtype=dtype, device=DEV)
    return raw, model, plain_config(raw), {k: v.float() for k, v in tensors.items()}


def prompt_lengths(kind, n_requests):
    # tiny B's window is 24: lengths on both sides of it; at 3B sizes (window 96) the first few
    # requests are long enough for the window to bite while they decode
    if kind == "B":
        cycle = [1, 3, 23, 24, 25, 40, 9, 17]
        return [cycle[i % len(cycle)] for i in range(n_requests)]
    long_ones = [110, 97, 85, 40]
    return [long_ones[i] if i < len(long_ones) else 3 + (5 * i) % 11 for i in range(n_requests)]


def run_case(kind, dtype, n_requests, expect_bucket):
    from matricxon_b200.engine.core import EngineCore
    from matricxon_b200.engine.step import StepEntry

    raw, model, cfg, weights = material(kind, dtype)
    vocab = raw["vocab_size"]
    generator = torch.Generator().manual_seed(100 + n_requests)
    lengths = prompt_lengths(kind, n_requests)
    sequences = [torch.randint(0, vocab, (n + DECODE_STEPS,), generator=generator).tolist() for n in lengths]
    core = EngineCore(model, max_cache_tokens=n_requests * 192, max_requests=n_requests, poison_cache=True)
    ids = [f"r{i}" for i in range(n_requests)]
    for rid in ids:
        core.cache.add_request(rid)
    # the prompts as one mixed eager step; then every request decodes in every step (the tokens are
    # given, not sampled, so that a wrong logit cannot hide behind the token it would have chosen)
    core.runner.run([StepEntry(rid, seq[:n], []) for rid, seq, n in zip(ids, sequences, lengths)])
    got = [[] for _ in ids]
    for step in range(DECODE_STEPS):
        entries = [StepEntry(rid, [seq[n + step]], [0]) for rid, seq, n in zip(ids, sequences, lengths)]
        logits = core.runner.run(entries)
        for i in range(n_requests):
            got[i].append(logits[i].clone())
    core.runner.check_status()
    if expect_bucket is None:
        assert not core.runner._graphs, "a step beyond the largest captured size must run eagerly"
    else:
        assert list(core.runner._graphs) == [expect_bucket]
    worst_ratio = 0.0
    for i, (seq, n) in enumerate(zip(sequences, lengths)):
        reference = plain_forward(cfg, weights, seq, dtype=torch.float32)[n:].numpy()
        mine = torch.stack(got[i]).cpu().numpy()
        limit = (2e-4 if dtype == "float32" else 0.03) * float(np.abs(reference).max())
        if kind == "B" and dtype == "float32":
            limit = 2e-5
        worst = np.abs(mine - reference).max(axis=1)
        bad = np.nonzero(worst > limit)[0]
        assert bad.size == 0, (f"request {i} (prompt {n}): first wrong decoded position {n + bad[0]}, "
                               f"error {worst[bad[0]]:.3e} > {limit:.2e}")
        worst_ratio = max(worst_ratio, float(worst.max() / limit))
    for rid in ids:
        core.cache.free_request(rid)
    core.cache.check_invariants()
    return worst_ratio


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_requests, bucket", [(24, 32), (64, 64), (70, None)])
def test_many_requests_decode_together_tiny_b(dtype, n_requests, bucket):
    run_case("B", dtype, n_requests, bucket)


@pytest.mark.parametrize("dtype, n_requests, bucket", [("bfloat16", 24, 32), ("bfloat16", 64, 64),
                                                       ("float32", 24, 32), ("bfloat16", 70, None)])
def test_many_requests_decode_together_3b_layer_sizes(dtype, n_requests, bucket):
    run_case("3b", dtype, n_requests, bucket)

"""StarCoder2-3B layer sizes (hidden 3072, 24 heads, 2 KV heads, head_dim 128, intermediate 12288,
vocabulary 49152, biases, tied head), two layers, random weights: the engine against the plain
implementation under every way of cutting the work, in float32 and in bfloat16. A window of 96
makes the sliding window bite inside a 200-token request."""

import numpy as np
import pytest
import torch

from plain_reference import plain_config, plain_forward

pytestmark = pytest.mark.gpu

RAW = {
    "model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 3072, "num_attention_heads": 24, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 49152, "rope_theta": 999999.4420358813,
    "sliding_window": 96, "max_position_embeddings": 16384, "norm_epsilon": 1e-5, "use_bias": True,
    "tie_word_embeddings": True, "hidden_act": "gelu_pytorch_tanh",
}
LENGTHS = {"a": 200, "b": 77, "c": 130}


@pytest.fixture(scope="module")
def material():
    from matricxon_b200.config.registry import config_from_dict
    from matricxon_b200.weights.random_init import RandomInit, random_tensors

    config = config_from_dict(dict(RAW))
    tensors = random_tensors(config, seed=3, init=RandomInit(0.02, 0.02, 0.0, 0.0), store_dtype=torch.bfloat16)
    generator = torch.Generator().manual_seed(9)
    prompts = {rid: torch.randint(0, RAW["vocab_size"], (n,), generator=generator).tolist()
               for rid, n in LENGTHS.items()}
    cfg = plain_config(RAW)
    weights = {k: v.float() for k, v in tensors.items()}
    reference = {rid: plain_forward(cfg, weights, ids, dtype=torch.float32).numpy() for rid, ids in prompts.items()}
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

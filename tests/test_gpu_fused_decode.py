"""The one-kernel decode step (csrc/decode_fused.cu) against the plain implementation and
against the part-by-part engine, at two configurations it takes (head_dim 64 and 128, with and
without window, bias, tied head; a vocabulary that is no multiple of 16; a feed-forward wider
than the kernel's activation stage) and at batch sizes on both sides of its 8-row tile."""

import numpy as np
import pytest
import torch

from plain_reference import plain_config, plain_forward

pytestmark = pytest.mark.gpu

FUSED_A = {
    "model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 352, "vocab_size": 1000, "rope_theta": 10000.0,
    "sliding_window": 40, "max_position_embeddings": 512, "norm_epsilon": 1e-5, "use_bias": True,
    "tie_word_embeddings": True, "hidden_act": "gelu_pytorch_tanh",
}
FUSED_B = {
    "model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 1,
    "head_dim": 128, "intermediate_size": 1312, "vocab_size": 777, "rope_theta": 100000.0,
    "sliding_window": None, "max_position_embeddings": 1024, "norm_epsilon": 1e-6, "use_bias": False,
    "tie_word_embeddings": False, "hidden_act": "gelu_pytorch_tanh",
}
CASES = {"A": (FUSED_A, 16, 5), "B": (FUSED_B, 32, 6)}          # config, page size, seed


def make(name):
    from matricxon_b200.config.registry import config_from_dict
    from matricxon_b200.weights.random_init import RandomInit, random_tensors

    raw, page_size, seed = CASES[name]
    config = config_from_dict(dict(raw))
    init = RandomInit(0.05, 0.05, 0.1, 0.1) if raw["use_bias"] else RandomInit(0.05, 0.0, 0.0, 0.0)
    tensors = random_tensors(config, seed=seed, init=init, store_dtype=torch.bfloat16)
    return raw, config, tensors, page_size


def decode_tail(replayer, prompts, tail):
    """Prompts minus their last ``tail`` tokens in one step each, then the tails one token per
    request and step (all requests side by side). Returns {(request, position): logits}."""
    logits = {}
    for rid, ids in prompts.items():
        head = ids[:len(ids) - tail]
        out = replayer.step([{"id": rid, "tokens": head, "want": list(range(len(head)))}], [])
        for i, row in enumerate(out.numpy()):
            logits[(rid, i)] = row
    for k in range(tail):
        entries = [{"id": rid, "tokens": [ids[len(ids) - tail + k]], "want": [0]} for rid, ids in prompts.items()]
        ended = list(prompts) if k == tail - 1 else []
        out = replayer.step(entries, ended)
        for (rid, ids), row in zip(prompts.items(), out.numpy()):
            logits[(rid, len(ids) - tail + k)] = row
    return logits


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("n_requests", [1, 3, 8, 11])
def test_fused_decode_matches_plain_and_parts(name, n_requests, monkeypatch):
    from matricxon_b200.engine.core import model_from_tensors
    from matricxon_b200.engine.replay import TraceReplayer

    raw, config, tensors, page_size = make(name)
    generator = torch.Generator().manual_seed(100 + n_requests)
    lengths = [70 + 23 * i for i in range(n_requests)]
    prompts = {f"r{i}": torch.randint(0, raw["vocab_size"], (n,), generator=generator).tolist()
               for i, n in enumerate(lengths)}
    tail = 36
    cfg = plain_config(raw)
    weights = {k: v.float() for k, v in tensors.items()}
    reference = {rid: plain_forward(cfg, weights, ids, dtype=torch.float32).numpy() for rid, ids in prompts.items()}

    results = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("MATRICXON_FUSED_DECODE", mode)
        model = model_from_tensors(config, tensors, dtype="bfloat16", device="cuda:0", page_size=page_size)
        replayer = TraceReplayer(None, "bfloat16", max_tokens=sum(lengths) + 64 * n_requests, model=model,
                                 poison_cache=True)
        assert (replayer.core.runner.fused is not None) == (mode == "1")
        results[mode] = decode_tail(replayer, prompts, tail)
        replayer.core.runner.check_status()
        assert sum(replayer.core.cache.free_pages()) == sum(p.num_pages for p in replayer.core.cache.pools)

    for rid, ids in prompts.items():
        ref = reference[rid]
        scale = float(np.abs(ref).max())
        for position in range(len(ids) - tail, len(ids)):
            fused, parts = results["1"][(rid, position)], results["0"][(rid, position)]
            assert np.isfinite(fused).all(), f"{rid} position {position}: the fused step gave a non-finite logit"
            error = float(np.abs(fused - ref[position]).max())
            assert error <= 0.03 * scale, f"{rid} position {position}: fused vs plain {error:.3e} > {0.03 * scale:.2e}"
            drift = float(np.abs(fused - parts).max())
            assert drift <= 0.02 * scale, f"{rid} position {position}: fused vs parts {drift:.3e}"


def test_fused_decode_declines_what_it_does_not_take(monkeypatch):
    """A model whose head_dim the kernel is not built for keeps the part-by-part path."""
    monkeypatch.setenv("MATRICXON_FUSED_DECODE", "1")
    from matricxon_b200.engine.core import model_from_tensors
    from matricxon_b200.engine.replay import TraceReplayer
    from tiny_configs import tiny_config, tiny_tensors

    model = model_from_tensors(tiny_config("A"), tiny_tensors("A", torch.bfloat16), dtype="bfloat16")
    replayer = TraceReplayer(None, "bfloat16", max_tokens=256, model=model)
    assert replayer.core.runner.fused is None

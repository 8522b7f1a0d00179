"""The plain implementation against the reference's own model code (stored golden logits)
and against itself (its parts, its masks)."""

import os

import numpy as np
import pytest
import torch

from plain_reference import (
    plain_attention_core,
    plain_forward,
    plain_config,
    plain_gelu_tanh,
    plain_layernorm,
    plain_mask,
    plain_sample,
    plain_top_k,
    plain_top_p,
)
from tiny_configs import TINY, random_ids, tiny_tensors

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
PROMPT_LENGTHS = {"A": 24, "B": 20}


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_model_code(name):
    """Logits of matricxon's Starcoder2Architecture (float32, CPU) on the same seeded weights."""
    golden = np.load(os.path.join(GOLDEN, f"reference_logits_{name}.npy"))
    raw = TINY[name][0]
    ids = random_ids(PROMPT_LENGTHS[name], raw["vocab_size"], seed=100 + ord(name))
    logits = plain_forward(plain_config(raw), tiny_tensors(name), ids, dtype=torch.float32)
    assert logits.shape == golden.shape
    assert np.abs(logits.numpy() - golden).max() < 1e-5
    logits64 = plain_forward(plain_config(raw), tiny_tensors(name), ids, dtype=torch.float64)
    assert np.abs(logits64.numpy() - golden).max() < 1e-5


def test_mask_rule():
    mask = plain_mask(q_len=3, kv_len=10, offset=7, window=4)
    # query 0 sits at position 7 and sees keys 4..7
    assert mask[0].nonzero().flatten().tolist() == [4, 5, 6, 7]
    assert mask[2].nonzero().flatten().tolist() == [6, 7, 8, 9]
    full = plain_mask(3, 10, 7, None)
    assert full[0].sum() == 8 and full[2].sum() == 10


def test_window_changes_logits_only_beyond_it():
    raw = dict(TINY["A"][0])
    weights = tiny_tensors("A")
    ids = random_ids(50, raw["vocab_size"], 5)
    windowed = plain_forward(plain_config(raw), weights, ids)
    raw["sliding_window"] = None
    full = plain_forward(plain_config(raw), weights, ids)
    assert torch.allclose(windowed[:32], full[:32], atol=1e-12)
    assert (windowed[40:] - full[40:]).abs().max() > 1e-6


def test_layernorm_matches_torch():
    x = torch.randn(5, 96, dtype=torch.float64)
    w, b = torch.randn(96, dtype=torch.float64), torch.randn(96, dtype=torch.float64)
    expected = torch.nn.functional.layer_norm(x, (96,), w, b, 1e-6)
    assert torch.allclose(plain_layernorm(x, w, b, 1e-6), expected, atol=1e-12)


def test_gelu_matches_torch():
    u = torch.linspace(-6, 6, 101, dtype=torch.float64)
    assert torch.allclose(plain_gelu_tanh(u), torch.nn.functional.gelu(u, approximate="tanh"), atol=1e-12)


def test_attention_core_gqa_matches_sdpa():
    torch.manual_seed(0)
    q = torch.randn(6, 9, 16, dtype=torch.float64)
    k = torch.randn(2, 9, 16, dtype=torch.float64)
    v = torch.randn(2, 9, 16, dtype=torch.float64)
    out = plain_attention_core(q, k, v, 16 ** -0.5, None)
    expected = torch.nn.functional.scaled_dot_product_attention(
        q[None], k[None].repeat_interleave(3, dim=1), v[None].repeat_interleave(3, dim=1),
        is_causal=True)[0]
    assert torch.allclose(out, expected, atol=1e-10)


def test_sampler_greedy_and_filters():
    logits = torch.tensor([0.1, 2.0, -1.0, 2.0, 0.5])
    assert plain_sample(logits, [], 0.0, 40, 0.9, 1.1, 0.3) == 1          # ties -> lowest index
    kept = plain_top_k(logits, 2)
    assert torch.isfinite(kept).tolist() == [False, True, False, True, False]
    kept = plain_top_p(torch.tensor([3.0, 1.0, 0.0, -2.0]), 0.5)
    assert torch.isfinite(kept).tolist() == [True, False, False, False]
    # repeat penalty pushes a generated token below the runner-up
    assert plain_sample(torch.tensor([1.0, 0.95]), [0], 0.0, 0, 1.0, 1.2, 0.0) == 1


def test_sampler_inverse_cdf_sweep():
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0])
    probs = torch.softmax(logits.double(), 0)
    counts = torch.zeros(4)
    n = 4000
    for i in range(n):
        counts[plain_sample(logits, [], 1.0, 0, 1.0, 1.0, (i + 0.5) / n)] += 1
    assert torch.allclose(counts / n, probs.float(), atol=2e-3)

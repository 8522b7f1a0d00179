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


# ------------------------------------------------------------------ the reference's own C kernels
def _golden_module():
    import importlib.util

    spec = importlib.util.spec_from_file_location("make_golden_native",
                                                  os.path.join(GOLDEN, "make_golden_native.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_window_mask_and_attention_match_the_reference_c_kernel():
    """``mx_attention`` (app/native/src/mx_attention.c:16-68) and ``_causal_mask``
    (app/architectures/gemma4_layers.py:17-34), run on the CPU by tests/golden/make_golden_native.py:
    the window rule of the plain implementation rests on their outputs, not on a reading."""
    golden = _golden_module()
    stored = np.load(os.path.join(GOLDEN, "native_attention.npz"))
    for index, case in enumerate(golden.ATTENTION_CASES):
        heads, kv_heads, dim, n_q, n_kv, offset, window = case
        q, k, v = golden.attention_inputs(index, case)
        mask = plain_mask(n_q, n_kv, offset, window or None)
        assert np.array_equal(mask.numpy(), stored[f"mask_{index}"]), case
        out = plain_attention_core(q.double(), k.double(), v.double(), dim ** -0.5, window or None, offset)
        assert np.abs(out.numpy() - stored[f"out_{index}"]).max() < 1e-5, case
        if window:
            # the window matters in these cases: without it the result differs
            full = plain_attention_core(q.double(), k.double(), v.double(), dim ** -0.5, None, offset)
            if offset + 1 > window:
                assert np.abs(full.numpy() - stored[f"out_{index}"]).max() > 1e-4, case


def test_sampler_matches_the_reference_c_kernel():
    """``mx_sample`` (app/native/src/mx_sample.c:51-108) over a sweep of uniforms. Without top-p
    the kernel draws in vocabulary order and the plain sampler picks the same token for every
    uniform (up to a boundary within rounding). With top-p below one the kernel sorts its
    candidates and draws in descending order (mx_sample.c:88-107) where this engine keeps
    vocabulary order, so there the kept set and each token's share of the draws are compared."""
    golden = _golden_module()
    stored = np.load(os.path.join(GOLDEN, "native_sampler.npz"))
    for index, case in enumerate(golden.SAMPLER_CASES):
        _, temperature, top_k, top_p, penalty, _ = case
        logits, generated = golden.sampler_inputs(index, case)
        theirs = stored[f"tokens_{index}"].tolist()
        ours = [plain_sample(logits, generated, temperature, top_k, top_p, penalty, (i + 0.5) / golden.SWEEP)
                for i in range(golden.SWEEP)]
        if top_p >= 1.0:
            assert sum(a != b for a, b in zip(ours, theirs)) <= 1, case
        else:
            assert set(ours) == set(theirs), case
            for token in set(theirs):
                assert abs(ours.count(token) - theirs.count(token)) <= 2, (case, token)

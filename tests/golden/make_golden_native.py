"""Runs nesmind/matricxon's own C kernels for attention and sampling, and its window mask, on
the CPU and stores small outputs beside this script (``native_attention.npz``,
``native_sampler.npz``).

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_native.py /path/to/reference

The reference's ``NativeKernelLibrary`` (app/native/library.py:58-103) compiles
``app/native/src/*.c`` into a temporary folder; its ``_NativeBackend``
(app/native/fused_ops.py:30-74) binds ``mx_attention`` (app/native/src/mx_attention.c:16-68)
and ``mx_sample`` (app/native/src/mx_sample.c:51-108). The mask is ``_causal_mask`` of
app/architectures/gemma4_layers.py:17-34. Inputs are drawn from seeds that the test repeats, so
only outputs are stored.
"""

import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

# (heads, kv heads, dim, n_q, n_kv, offset, window); window 0 = none. The first four are the
# shapes of the reference's own test (tests/unit/test_fused_ops.py:64-88); the others are the
# two tiny configurations' head geometries at their windows, with queries on both sides of the
# window's edge.
ATTENTION_CASES = [
    (4, 2, 16, 1, 40, 39, 8),
    (4, 2, 16, 4, 12, 8, 5),
    (4, 2, 16, 3, 40, 37, 0),
    (4, 2, 16, 1, 1, 0, 0),
    (4, 2, 16, 5, 70, 65, 32),      # tiny A: 4 heads, 2 KV heads, head_dim 16, window 32
    (4, 2, 16, 8, 36, 28, 32),      # queries at 28..35: the window's edge passes through them
    (3, 1, 32, 6, 60, 54, 24),      # tiny B: 3 heads, 1 KV head, head_dim 32, window 24
    (3, 1, 32, 4, 26, 22, 24),
]

# (vocab, temperature, top_k, top_p, penalty, number of generated ids)
SAMPLER_CASES = [
    (1000, 1.0, 0, 1.0, 1.0, 0),
    (1000, 0.7, 0, 1.0, 1.0, 0),
    (1000, 0.8, 40, 1.0, 1.1, 5),
    (512, 1.3, 5, 1.0, 1.5, 3),
    (512, 0.8, 40, 0.9, 1.1, 5),    # top-p below one: the kernel draws in sorted order, see the test
    (1000, 0.5, 7, 0.5, 1.0, 0),
]
SWEEP = 400


def attention_inputs(case_index: int, case):
    heads, kv_heads, dim, n_q, n_kv, _, _ = case
    generator = torch.Generator().manual_seed(1000 + case_index)
    q = torch.randn(heads, n_q, dim, generator=generator)
    k = torch.randn(kv_heads, n_kv, dim, generator=generator)
    v = torch.randn(kv_heads, n_kv, dim, generator=generator)
    return q, k, v


def sampler_inputs(case_index: int, case):
    vocab, _, _, _, _, n_generated = case
    generator = torch.Generator().manual_seed(2000 + case_index)
    logits = torch.randn(vocab, generator=generator) * 2.0
    generated = torch.randint(0, vocab, (n_generated,), generator=generator).tolist()
    if n_generated:
        generated[0] = int(torch.argmax(logits))     # the penalty should move the favourite
    return logits, generated


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden_native.py <path to a checkout of nesmind/matricxon>")
    sys.path.insert(0, sys.argv[1])
    from app.architectures.gemma4_layers import _causal_mask
    from app.native.fused_ops import _NativeBackend
    from app.native.library import NativeKernelLibrary

    with tempfile.TemporaryDirectory() as build_dir:
        backend = _NativeBackend(NativeKernelLibrary(build_dir=Path(build_dir)).load(), 1)
        stored = {}
        for index, case in enumerate(ATTENTION_CASES):
            heads, kv_heads, dim, n_q, n_kv, offset, window = case
            q, k, v = attention_inputs(index, case)
            out = torch.empty_like(q)
            backend.attention(q, k, v, out, dim ** -0.5, offset, window)
            stored[f"out_{index}"] = out.numpy()
            stored[f"mask_{index}"] = _causal_mask(n_q, n_kv, offset, window or None).numpy()
        np.savez(HERE / "native_attention.npz", **stored)
        print("attention:", len(ATTENTION_CASES), "cases")

        stored = {}
        for index, case in enumerate(SAMPLER_CASES):
            _, temperature, top_k, top_p, penalty, _ = case
            logits, generated = sampler_inputs(index, case)
            ids = torch.tensor(sorted(set(generated)) if penalty != 1.0 else [], dtype=torch.int32)
            tokens = [backend.sample(logits, ids, penalty, temperature, top_k, top_p, (i + 0.5) / SWEEP)
                      for i in range(SWEEP)]
            stored[f"tokens_{index}"] = np.asarray(tokens, dtype=np.int32)
        np.savez(HERE / "native_sampler.npz", **stored)
        print("sampler:", len(SAMPLER_CASES), "cases of", SWEEP, "uniforms")


if __name__ == "__main__":
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    main()

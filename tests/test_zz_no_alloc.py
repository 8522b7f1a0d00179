"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of this library may not allocate device memory while they run (a plugin inside
another framework's memory pool, a latency-bound loop that must avoid the allocator's locks
and implicit synchronisation, a process with a memory budget fixed at start-up). For them
``mx_paged_attention_static`` keeps the split-key scratch in an 8 MiB array inside the
library. This test calls it with raw pointers, twice in a row on different inputs (the
array keeps the first call's partials), and checks each output against the ordinary entry
point, which takes its scratch from the caller. It is collected last on purpose.
"""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def static_entry():
    from matricxon_b200.ops.library import library

    lib = library()
    fn = lib.mx_paged_attention_static
    fn.argtypes = [c_void_p, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p,
                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int,
                   c_void_p, c_void_p]
    fn.restype = c_int
    lib.mx_static_attention_scratch_bytes.restype = c_longlong
    lib.mx_static_attention_scratch_bytes.argtypes = []
    return lib, fn


def call_static(fn, q, cache, tables, tok_seq, positions, heads, kv_heads, dim, window, scale, n_splits,
                out_cols=None):
    from matricxon_b200.ops.kernels import dtype_code

    n = q.shape[0]
    out = torch.full((n, out_cols or heads * dim), float("nan"), dtype=q.dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    code = fn(q.data_ptr(), dtype_code(q.dtype), q.stride(0), cache.data_ptr(), cache.shape[0],
              cache.shape[3], tables.data_ptr(), tables.stride(0), tok_seq.data_ptr(),
              positions.data_ptr(), n, heads, kv_heads, dim, window or 0, scale, out.data_ptr(),
              out.stride(0), n_splits, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return code, out, int(status.item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_attention_matches_the_ordinary_entry_point_twice(dtype):
    from test_gpu_kernels import paged_case, run_attention

    from matricxon_b200.ops import kernels

    lib, fn = static_entry()
    assert lib.mx_static_attention_scratch_bytes() == 8 * 1024 * 1024
    tolerance = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    from test_gpu_kernels import reference_attention

    first = dict(heads=24, kv_heads=2, dim=128, page=16, lens=[700, 333, 90], q=[1, 1, 3], window=256, splits=8, seed=1)
    # the third call has the first one's shapes with more splits, right after a call that left
    # other partials in the array: a merge that read a split it had not written would show
    cases = [first, dict(heads=6, kv_heads=3, dim=64, page=16, lens=[150, 41], q=[2, 1], window=None, splits=5, seed=2),
             dict(first, splits=16, seed=4)]
    for case in cases:                                    # back to back: the array is not cleared
        q, cache, tables, tok_seq, positions, dense = paged_case(
            dtype, case["heads"], case["kv_heads"], case["dim"], case["page"], case["lens"], case["q"],
            seed=case["seed"])
        scale = case["dim"] ** -0.5
        plain = reference_attention(dense, case["q"], case["lens"], scale, case["window"])
        expected, st = run_attention(kernels, q, cache, tables, tok_seq, positions, case["heads"],
                                     case["kv_heads"], case["dim"], case["window"], scale, case["splits"])
        assert st == 0
        code, got, st = call_static(fn, q, cache, tables, tok_seq, positions, case["heads"],
                                    case["kv_heads"], case["dim"], case["window"], scale, case["splits"])
        assert code == 0 and st == 0
        assert not torch.isnan(got).any()
        assert torch.allclose(got.float(), expected.float(), **tolerance)
        # and against the plain attention itself, not only against the sibling entry point
        assert torch.allclose(got.double().cpu(), plain, **tolerance)


def test_static_scratch_attention_refuses_what_does_not_fit():
    from test_gpu_kernels import paged_case

    lib, fn = static_entry()
    # 1,100 tokens x 24 heads x 4 splits x 130 floats > 8 MiB
    q, cache, tables, tok_seq, positions, _ = paged_case(torch.bfloat16, 24, 2, 128, 16, [1100], [1100], seed=3)
    code, out, st = call_static(fn, q, cache, tables, tok_seq, positions, 24, 2, 128, None, 0.1, 4)
    assert code == -1 and torch.isnan(out.float()).all()           # nothing was launched
    message = lib.mx_last_error_message().decode()
    assert "built-in array holds 8388608" in message
    code, out, st = call_static(fn, q, cache, tables, tok_seq, positions, 24, 2, 128, None, 0.1, 1)
    assert code == 0 and st == 0 and not torch.isnan(out.float()).any()   # one split needs no scratch
    # sizes that make no sense are refused before they are multiplied into a byte count
    for heads, kv_heads, dim, splits in ((0, 2, 128, 4), (-24, 2, 128, 4), (24, 5, 128, 4), (24, 2, -128, 4),
                                         (24, 2, 24, 4), (24, 2, 128, 70000), (24, 2, 128, 0)):
        code, out, st = call_static(fn, q, cache, tables, tok_seq, positions, heads, kv_heads, dim, None, 0.1, splits,
                                    out_cols=24 * 128)
        assert code == -1 and torch.isnan(out.float()).all(), (heads, kv_heads, dim, splits)

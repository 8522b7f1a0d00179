"""The streaming product for up to 128 rows (TMA + tcgen05 with the tokens as the narrow side)
against a float64 product: every epilogue, row counts on both sides of the 16-token padding, widths
that deal out unevenly over the SMs, a K that is no multiple of 64, a vocabulary-sized N that gives
every block several tiles, and rows that must not depend on their neighbours."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def gelu_tanh(u):
    return 0.5 * u * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (u + 0.044715 * u ** 3)))


def run(k, m, n, k_dim, mode, seed=0, with_bias=True):
    torch.manual_seed(seed + m + n)
    a = torch.randn(m, k_dim, device=DEV).bfloat16()
    w = (torch.randn(n, k_dim, device=DEV) / math.sqrt(k_dim)).bfloat16()
    bias = torch.randn(n, device=DEV) if with_bias else None
    residual = torch.randn(m, n, device=DEV) if mode == k.EPILOGUE_RESIDUAL else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    f32 = mode in (k.EPILOGUE_RESIDUAL, k.EPILOGUE_F32)
    out = torch.full((m + 1, n), float("nan"), dtype=torch.float32 if f32 else torch.bfloat16, device=DEV)
    k.gemm_stream(a, w, bias, residual, out[:m], mode, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.isnan(out[m].float()).all()                 # nothing written beyond the last row
    acc = a.double() @ w.double().T
    if with_bias:
        acc = acc + bias.double()
    if mode == k.EPILOGUE_GELU:
        acc = gelu_tanh(acc)
    if mode == k.EPILOGUE_RESIDUAL:
        acc = acc + residual.double()
    return out[:m].double(), acc, a, w, bias


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("m", [1, 8, 16, 17, 33, 64, 100, 128])
@pytest.mark.parametrize("n,k_dim", [(3584, 3072), (1000, 96), (50, 352), (17, 32), (3072, 1024), (5000, 200)])
def test_streaming_gemm_every_epilogue(mode, m, n, k_dim):
    from matricxon_b200.ops import kernels as k

    got, want, *_ = run(k, m, n, k_dim, mode)
    bf16_out = mode in (k.EPILOGUE_NONE, k.EPILOGUE_GELU)
    tolerance = dict(atol=3e-2, rtol=2e-2) if bf16_out else dict(atol=2e-3, rtol=2e-3)
    worst = (got - want).abs().max()
    assert torch.allclose(got, want, **tolerance), (float(worst), torch.nonzero((got - want).abs() > 0.1)[:4].tolist())


@pytest.mark.parametrize("m", [3, 64])
def test_streaming_gemm_long_k_and_vocabulary_width(m):
    from matricxon_b200.ops import kernels as k

    got, want, *_ = run(k, m, 3072, 12288, k.EPILOGUE_RESIDUAL, seed=1)
    assert torch.allclose(got, want, atol=4e-3, rtol=2e-3), float((got - want).abs().max())
    got, want, *_ = run(k, m, 49152, 3072, k.EPILOGUE_F32, seed=2, with_bias=False)      # several tiles per block
    assert torch.allclose(got, want, atol=4e-3, rtol=2e-3), float((got - want).abs().max())
    got, want, *_ = run(k, m, 49153, 1024, k.EPILOGUE_F32, seed=3, with_bias=False)      # a width that is odd
    assert torch.allclose(got, want, atol=4e-3, rtol=2e-3), float((got - want).abs().max())


def test_a_row_does_not_depend_on_the_rows_beside_it():
    from matricxon_b200.ops import kernels as k

    torch.manual_seed(5)
    a = torch.randn(64, 3072, device=DEV).bfloat16()
    w = (torch.randn(3584, 3072, device=DEV) / 55).bfloat16()
    bias = torch.randn(3584, device=DEV)
    together = torch.empty(64, 3584, dtype=torch.bfloat16, device=DEV)
    k.gemm_stream(a, w, bias, None, together, k.EPILOGUE_GELU)
    for rows in ([0], [5, 6, 7], list(range(40, 57))):
        alone = torch.empty(len(rows), 3584, dtype=torch.bfloat16, device=DEV)
        k.gemm_stream(a[rows].contiguous(), w, bias, None, alone, k.EPILOGUE_GELU)
        assert torch.equal(alone, together[rows])


def test_streaming_gemm_refuses_what_it_cannot_take():
    from matricxon_b200.ops import kernels as k
    from matricxon_b200.ops.library import KernelLibraryError

    w = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros(129, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(KernelLibraryError, match="at most 128"):
        k.gemm_stream(torch.zeros(129, 64, device=DEV, dtype=torch.bfloat16), w, None, None, out, 0)
    w = torch.zeros(64, 36, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(KernelLibraryError, match="multiple of 8"):
        k.gemm_stream(torch.zeros(4, 36, device=DEV, dtype=torch.bfloat16), w, None, None, out[:4], 0)

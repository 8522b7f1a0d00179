"""The TMA + tcgen05 matrix product against float64, at sizes that fill no tile, with every epilogue."""

import math

import pytest
import torch

from plain_reference import plain_gelu_tanh

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("m,n,k_dim", [(128, 256, 64), (200, 1000, 96), (129, 257, 64), (17, 130, 352),
                                       (300, 3072, 1024), (2048, 3584, 3072), (1000, 96, 12288)])
def test_tcgen05_gemm_all_epilogues(m, n, k_dim):
    from matricxon_b200.ops import kernels as k

    torch.manual_seed(m + n + k_dim)
    a = torch.randn(m, k_dim, device=DEV).bfloat16()
    w = (torch.randn(n, k_dim, device=DEV) / math.sqrt(k_dim)).bfloat16()
    bias = torch.randn(n, device=DEV)
    residual = torch.randn(m, n, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert k.tcgen05_gemm_supported(a, w)
    acc = (a.double() @ w.double().T + bias.double()).cpu()
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_tcgen05(a, w, bias, None, out, k.EPILOGUE_NONE, status)
    assert status.item() == 0
    assert torch.allclose(out.double().cpu(), acc, atol=2e-2, rtol=2e-2)
    k.gemm_tcgen05(a, w, bias, None, out, k.EPILOGUE_GELU, status)
    assert torch.allclose(out.double().cpu(), plain_gelu_tanh(acc), atol=2e-2, rtol=2e-2)
    out32 = residual.clone()
    k.gemm_tcgen05(a, w, bias, out32, out32, k.EPILOGUE_RESIDUAL, status)          # in place
    assert torch.allclose(out32.double().cpu(), acc + residual.double().cpu(), atol=2e-3, rtol=1e-4)
    out32.fill_(float("nan"))
    k.gemm_tcgen05(a, w, None, None, out32, k.EPILOGUE_F32, status)
    assert torch.allclose(out32.double().cpu(), acc - bias.double().cpu(), atol=2e-3, rtol=1e-4)
    assert status.item() == 0


@pytest.fixture
def forced_tiles():
    from matricxon_b200.ops import kernels as k

    yield k.gemm_tcgen05_force_tiles
    k.gemm_tcgen05_force_tiles(0)


@pytest.mark.parametrize("rows", [128, 256, 512])
@pytest.mark.parametrize("m,n,k_dim", [(513, 264, 64), (700, 3000, 256), (1537, 3072, 1024), (1100, 1000, 96),
                                       (200, 1000, 3072), (300, 3072, 12288)])
def test_tcgen05_gemm_every_tile_height(rows, m, n, k_dim, forced_tiles):
    """The three kernels (128-row tiles, 256-row tiles, 512-row tiles on pairs of SMs) on the same
    products: each is forced in turn; edges in M, N and K, an N that is no multiple of 16. With a
    residual added in place the 256-row kernel shares K out between blocks (the long-K cases)."""
    from matricxon_b200.ops import kernels as k

    forced_tiles(rows)
    torch.manual_seed(rows + m)
    a = torch.randn(m, k_dim, device=DEV).bfloat16()
    w = (torch.randn(n, k_dim, device=DEV) / math.sqrt(k_dim)).bfloat16()
    bias = torch.randn(n, device=DEV)
    residual = torch.randn(m, n, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    acc = (a.double() @ w.double().T + bias.double()).cpu()
    out = torch.full((m + 1, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_tcgen05(a, w, bias, None, out[:m], k.EPILOGUE_GELU, status)
    assert torch.allclose(out[:m].double().cpu(), plain_gelu_tanh(acc), atol=2e-2, rtol=2e-2)
    assert torch.isnan(out[m]).all()                                   # nothing written past the last row
    out32 = residual.clone()
    k.gemm_tcgen05(a, w, bias, out32, out32, k.EPILOGUE_RESIDUAL, status)          # in place
    assert torch.allclose(out32.double().cpu(), acc + residual.double().cpu(), atol=2e-3, rtol=1e-4)
    apart = torch.full((m, n), float("nan"), device=DEV)
    k.gemm_tcgen05(a, w, bias, residual, apart, k.EPILOGUE_RESIDUAL, status)       # residual elsewhere
    assert torch.allclose(apart.double().cpu(), acc + residual.double().cpu(), atol=2e-3, rtol=1e-4)
    k.gemm_tcgen05(a, w, None, None, apart, k.EPILOGUE_F32, status)
    assert torch.allclose(apart.double().cpu(), acc - bias.double().cpu(), atol=2e-3, rtol=1e-4)
    assert status.item() == 0


def test_tcgen05_gemm_strided_rows_and_same_result_for_a_row_in_any_batch():
    from matricxon_b200.ops import kernels as k

    torch.manual_seed(0)
    wide = torch.randn(300, 3584, device=DEV).bfloat16()
    a = wide[:, 512:512 + 3072]                       # rows of a wider buffer
    w = (torch.randn(640, 3072, device=DEV) / 50).bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(300, 640, device=DEV)
    k.gemm_tcgen05(a, w, None, None, out, k.EPILOGUE_F32, status)
    ref = (a.double() @ w.double().T).cpu()
    assert torch.allclose(out.double().cpu(), ref, atol=2e-3, rtol=1e-4)
    part = torch.empty(40, 640, device=DEV)
    k.gemm_tcgen05(a[130:170], w, None, None, part, k.EPILOGUE_F32, status)
    assert torch.equal(part, out[130:170]) and status.item() == 0

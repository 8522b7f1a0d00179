"""``out = epilogue(x @ W.T + bias)``: the one matrix product every part uses.

Backends, chosen by the runtime:
  "simt"    -- the engine's own FP32-core kernel; the only backend of the 32-bit path.
  "skinny"  -- the engine's tensor-core kernel for at most 16 rows (decoding): the weight
               matrix is streamed once and the epilogue is fused.
  "tcgen05" -- the engine's TMA + tcgen05 kernel for prompt-sized products: operands staged by
               TMA, accumulator in tensor memory, epilogue fused.
  "library" -- cuBLAS through ``torch.mm`` for bfloat16 (the reference runs its products
               through nn.Linear, i.e. the library: app/architectures/qwen_layers.py:50-53),
               followed by the engine's fused bias / GELU / residual epilogue kernel.
  "auto"    -- "simt" for float32; for bfloat16 "skinny" up to 16 rows, "tcgen05" above 128 rows,
               and "library" between (a weight stream that 128-row tiles would leave to a few
               SMs) and for shapes neither takes (a K that is no multiple of 8).
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.kernels import (
    EPILOGUE_F32,
    EPILOGUE_GELU,
    EPILOGUE_NONE,
    EPILOGUE_RESIDUAL,
)
from matricxon_b200.ops.library import KernelLibraryError

_HAS_OUT_DTYPE: bool | None = None


def _mm_f32(x: torch.Tensor, w_t: torch.Tensor) -> torch.Tensor | None:
    """bfloat16 x bfloat16 with the float accumulator kept, when torch offers it."""
    global _HAS_OUT_DTYPE
    if _HAS_OUT_DTYPE is False:
        return None
    try:
        out = torch.mm(x, w_t, out_dtype=torch.float32)
        _HAS_OUT_DTYPE = True
        return out
    except (TypeError, RuntimeError):
        _HAS_OUT_DTYPE = False
        return None


def resolve_backend(requested: str, dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        if requested not in ("auto", "simt"):
            raise KernelLibraryError(
                f"the float32 path runs on the FP32-core kernel only, not {requested!r}")
        return "simt"
    if requested not in ("auto", "simt", "skinny", "tcgen05", "library"):
        raise KernelLibraryError(f"unknown GEMM backend {requested!r}")
    return requested


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, mode: int,
           residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
           backend: str = "auto") -> torch.Tensor:
    """x [M, K], weight [N, K] in the compute dtype; bias float32 [N] or None.

    mode EPILOGUE_NONE / EPILOGUE_GELU give the compute dtype; EPILOGUE_RESIDUAL
    (``residual + x @ W.T + bias``) and EPILOGUE_F32 give float32.
    """
    m, n = x.shape[0], weight.shape[0]
    out_dtype = torch.float32 if mode in (EPILOGUE_RESIDUAL, EPILOGUE_F32) else x.dtype
    backend = resolve_backend(backend, x.dtype)
    if backend == "auto":
        if kernels.skinny_gemm_supported(x, weight):
            backend = "skinny"
        elif m > 128 and kernels.tcgen05_gemm_supported(x, weight):
            backend = "tcgen05"
        else:
            backend = "library"
    if backend == "library" and out is None and mode == EPILOGUE_F32 and bias is None and m > 0:
        acc = _mm_f32(x, weight.t())
        if acc is not None:
            return acc
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    if m == 0:
        return out
    if backend == "simt":
        kernels.gemm_simt(x, weight, bias, residual, out, mode)
        return out
    if backend == "skinny":
        kernels.gemm_skinny(x, weight, bias, residual, out, mode)
        return out
    if backend == "tcgen05":
        kernels.gemm_tcgen05(x, weight, bias, residual, out, mode)
        return out
    # the library product keeps its float accumulator for every mode, so that bias, GELU and the
    # residual see the same unrounded sum as in the engine's own kernels
    acc = _mm_f32(x, weight.t())
    if acc is None:
        acc = torch.mm(x, weight.t())
    if mode == EPILOGUE_F32 and bias is None and acc.dtype == torch.float32:
        out.copy_(acc)
        return out
    kernels.epilogue(acc, bias, residual, out, mode)
    return out


__all__ = ["linear", "resolve_backend", "EPILOGUE_NONE", "EPILOGUE_GELU", "EPILOGUE_RESIDUAL",
           "EPILOGUE_F32"]

"""``out = epilogue(x @ W.T + bias)``: the one matrix product every part uses.

Backends, chosen by the runtime:
  "simt"    -- the engine's own FP32-core kernel; the only backend of the 32-bit path.
  "skinny"  -- the engine's tensor-core kernel for at most 16 rows (decoding): the weight
               matrix is streamed once and the epilogue is fused.
  "stream"  -- the engine's TMA + tcgen05 kernel for at most 128 rows with the tokens as the
               narrow side of the product: one block per SM streams its share of the weight rows.
  "tcgen05" -- the engine's TMA + tcgen05 kernel for prompt-sized products: operands staged by
               TMA, accumulator in tensor memory, epilogue fused.
  "library" -- cuBLAS through ``torch.mm`` for bfloat16 (the reference runs its products
               through nn.Linear, i.e. the library: app/architectures/qwen_layers.py:50-53),
               followed by the engine's fused bias / GELU / residual epilogue kernel.
  "auto"    -- "simt" for float32; for bfloat16 "skinny" up to 16 rows, "tcgen05" above 256 rows,
               "library" between (a weight stream that 128-row tiles would leave to a few SMs) and
               for shapes neither takes (a K that is no multiple of 8), and "stream" from 9 rows
               on where every SM owns many weight rows (``_pick`` gives the measured thresholds).
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
    if requested not in ("auto", "simt", "skinny", "stream", "tcgen05", "library"):
        raise KernelLibraryError(f"unknown GEMM backend {requested!r}")
    return requested


def _pick(x: torch.Tensor, weight: torch.Tensor, m: int, n: int) -> str:
    """The backend "auto" stands for, from measurements on B200 with weights streaming from HBM.
    Up to 8 rows the 16-row kernel is the fastest on every shape (its many small blocks hide the
    latencies that the streaming kernel's one pipeline per SM has to sit through). From 9 rows on that
    kernel works on two token blocks and slows by 40 %; the streaming kernel does not, and wins where
    every SM owns enough weight rows to keep its pipeline busy: 64 for 9 to 16 rows (the wide
    feed-forward matrix: 17 against 23 us; the vocabulary-sized head: 53 against 71 us), 256 for 17 to
    128 rows (the head: 59 against 66 us for the library's product plus the epilogue kernel)."""
    if 9 <= m <= 128 and kernels.stream_gemm_supported(x, weight):
        rows_per_block = -(-n // kernels.sm_count(x.device))
        if rows_per_block >= (64 if m <= 16 else 256):
            return "stream"
    if kernels.skinny_gemm_supported(x, weight):
        return "skinny"
    # up to 256 rows a product has one row of 256-row tiles and too few of them for 148 SMs (each is
    # bound by what one SM takes in through TMA): the library is faster there (73 against 86 us for
    # the four products of a layer at 256 rows; 104 against 114 at 512, where the long-K product
    # already favours the engine's kernel)
    # ... and up to 1,023 rows for products that are short in both N and K (the QKV and output
    # projections: 14 against 23 and 14 against 18 us at 512 rows), which have too few tiles to fill
    # the GPU and too little K to share out
    if m > 256 and kernels.tcgen05_gemm_supported(x, weight) and (m >= 1024 or n >= 8192 or x.shape[1] >= 8192):
        return "tcgen05"
    return "library"


class PendingSum:
    """``residual + x @ W.T + bias`` not yet added up: the library's float product of a step with 17 or
    more rows, handed to the norm that follows, which forms the sum on its way through the rows
    (``kernels.layernorm_sum``) instead of an epilogue pass of its own. ``tensor()`` adds it up for
    anybody else."""

    def __init__(self, acc: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor) -> None:
        self.acc, self.bias, self.residual = acc, bias, residual
        self._done = False

    @property
    def shape(self):
        return self.residual.shape

    @property
    def device(self):
        return self.residual.device

    @property
    def dtype(self):
        return self.residual.dtype

    def added_by_kernel(self) -> torch.Tensor:
        """For the kernel that adds the sum itself: the residual, which then holds it."""
        self._done = True
        return self.residual

    def tensor(self) -> torch.Tensor:
        if not self._done:
            kernels.epilogue(self.acc, self.bias, self.residual, self.residual, EPILOGUE_RESIDUAL)
            self._done = True
        return self.residual


def chosen_backend(x: torch.Tensor, weight: torch.Tensor, requested: str = "auto") -> str:
    """The backend ``linear`` would run this product on."""
    backend = resolve_backend(requested, x.dtype)
    return _pick(x, weight, x.shape[0], weight.shape[0]) if backend == "auto" else backend


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, mode: int,
           residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
           backend: str = "auto", defer_sum: bool = False) -> "torch.Tensor | PendingSum":
    """x [M, K], weight [N, K] in the compute dtype; bias float32 [N] or None.

    mode EPILOGUE_NONE / EPILOGUE_GELU give the compute dtype; EPILOGUE_RESIDUAL
    (``residual + x @ W.T + bias``) and EPILOGUE_F32 give float32.

    ``defer_sum`` (EPILOGUE_RESIDUAL into the residual itself): where the product is the library's, the
    caller gets a ``PendingSum`` instead of the sum and hands it to a norm that adds as it reads.
    """
    m, n = x.shape[0], weight.shape[0]
    out_dtype = torch.float32 if mode in (EPILOGUE_RESIDUAL, EPILOGUE_F32) else x.dtype
    backend = resolve_backend(backend, x.dtype)
    if backend == "auto":
        backend = _pick(x, weight, m, n)
    if backend == "library" and out is None and mode == EPILOGUE_F32 and bias is None and m > 0:
        acc = _mm_f32(x, weight.t())
        if acc is not None:
            return acc
    if (defer_sum and backend == "library" and mode == EPILOGUE_RESIDUAL and out is residual
            and residual is not None and m > 0):
        acc = _mm_f32(x, weight.t())
        if acc is not None:
            return PendingSum(acc, bias, residual)
    if backend == "library" and out is None and mode == EPILOGUE_NONE and bias is None and m > 0:
        return torch.mm(x, weight.t())        # nothing to add: the library's result is the result
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
    if backend == "stream":
        kernels.gemm_stream(x, weight, bias, residual, out, mode)
        return out
    if backend == "tcgen05":
        kernels.gemm_tcgen05(x, weight, bias, residual, out, mode)
        return out
    # Float outputs keep the library's float accumulator. Outputs in bfloat16 (the QKV product, the
    # feed-forward's first product) take the library's bfloat16 result and are rounded a second time
    # after bias and GELU: keeping the accumulator there too measured 4 % of a 64-row decode step (a
    # float pass over the widest activations), for a difference of one rounding in 2^-9.
    acc = None
    if out_dtype == torch.float32:
        acc = _mm_f32(x, weight.t())
    if acc is None:
        acc = torch.mm(x, weight.t())
    if mode == EPILOGUE_F32 and bias is None and acc.dtype == torch.float32:
        out.copy_(acc)
        return out
    kernels.epilogue(acc, bias, residual, out, mode)
    return out


__all__ = ["linear", "chosen_backend", "PendingSum", "resolve_backend", "EPILOGUE_NONE", "EPILOGUE_GELU", "EPILOGUE_RESIDUAL",
           "EPILOGUE_F32"]

"""Device time of the tcgen05 matrix product alone on the four products of a StarCoder2-3B layer.

    python -m matricxon_b200.ops.gemm_bench [rows [tile_rows [product]]]

``rows`` prompt tokens (default 2048); ``tile_rows`` forces one of the three kernels (128, 256, or 512
for the kernel on pairs of SMs; default: the library's own choice); ``product`` is one of qkv, o,
c_fc, c_proj (default: all). 40 launches timed with CUDA events after 4 warm-up launches, the weight
rotating over four copies. With the library built with ``MATRICXON_NVCC_EXTRA=-DTC_PROFILE`` the
cycles that the roles of the 256- and 512-row kernels spend in each phase are printed too.
"""
import ctypes
import math
import os
import sys

import torch

from matricxon_b200.ops import kernels as k
from matricxon_b200.ops.library import library

DEV = "cuda:0"
PRODUCTS = {"qkv": (3584, 3072, k.EPILOGUE_NONE), "o": (3072, 3072, k.EPILOGUE_RESIDUAL),
            "c_fc": (12288, 3072, k.EPILOGUE_GELU), "c_proj": (3072, 12288, k.EPILOGUE_RESIDUAL)}
MARKS = ["setup", "producer waits for a free stage", "issuer waits for the accumulator", "issuer waits for operands",
         "  of which a tile's first slice", "issuer, accumulator free to last commit", "epilogue waits for the accumulator",
         "epilogue drains", "whole block", None, "  drain: waits for tensor memory", "  drain: into shared memory",
         "  drain: out to global memory"]


def run(name, m):
    n, kd, mode = PRODUCTS[name]
    torch.manual_seed(0)
    a = torch.randn(m, kd, device=DEV).bfloat16()
    ws = [(torch.randn(n, kd, device=DEV) / math.sqrt(kd)).bfloat16() for _ in range(4)]
    bias = torch.randn(n, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    if mode == k.EPILOGUE_RESIDUAL:
        out = torch.randn(m, n, device=DEV)
        residual = out
    else:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        residual = None
    for i in range(4):
        k.gemm_tcgen05(a, ws[i], bias, residual, out, mode, status)
    torch.cuda.synchronize()
    marks = getattr(library(), "mx_gemm_tcgen05_marks", None) if "TC_PROFILE" in os.environ.get(
        "MATRICXON_NVCC_EXTRA", "") else None
    if marks is not None:
        marks.argtypes = [ctypes.c_void_p, ctypes.c_int]
        marks(None, 1)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 40
    start.record()
    for i in range(reps):
        k.gemm_tcgen05(a, ws[i % 4], bias, residual, out, mode, status)
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1000 / reps
    print(f"{name:7s} M {m} N {n} K {kd}: {us:7.1f} us  {2.0 * m * n * kd / us / 1e6:6.0f} TFLOP/s  status {status.item()}")
    if marks is not None:
        buf = (ctypes.c_ulonglong * 16)()
        marks(buf, 1)
        blocks = max(buf[9], 1)
        mhz = torch.cuda.clock_rate() if hasattr(torch.cuda, "clock_rate") else 1900
        for i, label in enumerate(MARKS):
            if label is not None and buf[i]:
                print(f"    {label:42s} {buf[i] / blocks / mhz:8.2f} us per block (at {mhz} MHz)")


if __name__ == "__main__":
    rows = int(sys.argv[1]) if len(sys.argv) > 1 else 2048
    if len(sys.argv) > 2 and sys.argv[2] != "auto":
        os.environ["MATRICXON_GEMM_TILES"] = sys.argv[2]
    for product in ([sys.argv[3]] if len(sys.argv) > 3 else list(PRODUCTS)):
        run(product, rows)

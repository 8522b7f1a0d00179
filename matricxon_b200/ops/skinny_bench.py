"""Device time of the decode-sized products with weights that stream from HBM.

    python -m matricxon_b200.ops.skinny_bench [rows]

The four products of a StarCoder2-3B layer and the output head at ``rows`` (default 8) decode rows. Every
launch reads another copy of the weight matrix (copies of 500-700 MB in total, several times the L2), inside
one CUDA graph, timed with CUDA events around five replays.
"""
import math
import sys

import torch

from matricxon_b200.ops import kernels as k

DEV = "cuda:0"


def run(name, rows, n, kd, mode):
    copies = max(2, int(700e6 // (n * kd * 2)))
    ws = [(torch.randn(n, kd, device=DEV) / math.sqrt(kd)).bfloat16() for _ in range(copies)]
    x = torch.randn(rows, kd, device=DEV).bfloat16()
    bias = torch.randn(n, device=DEV)
    if mode in (k.EPILOGUE_RESIDUAL, k.EPILOGUE_F32):
        out = torch.zeros(rows, n, device=DEV)
        residual = out if mode == k.EPILOGUE_RESIDUAL else None
    else:
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=DEV)
        residual = None
    reps = 4 * copies
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(3):
            k.gemm_skinny(x, ws[i % copies], bias, residual, out, mode)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(reps):
                k.gemm_skinny(x, ws[i % copies], bias, residual, out, mode)
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(5):
            graph.replay()
        end.record(stream)
        torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1000 / (5 * reps)
    mbytes = n * kd * 2 / 1e6
    print(f"{name:7s} rows {rows} N {n:6d} K {kd:6d}: {us:7.2f} us  {mbytes / us:5.2f} TB/s  "
          f"({copies} copies of {mbytes:.1f} MB)", flush=True)


if __name__ == "__main__":
    rows = int(sys.argv[1]) if len(sys.argv) > 1 else 8
    for name, n, kd, mode in [("qkv", 3584, 3072, k.EPILOGUE_NONE), ("o", 3072, 3072, k.EPILOGUE_RESIDUAL),
                              ("c_fc", 12288, 3072, k.EPILOGUE_GELU), ("c_proj", 3072, 12288, k.EPILOGUE_RESIDUAL),
                              ("head", 49152, 3072, k.EPILOGUE_F32)]:
        run(name, rows, n, kd, mode)

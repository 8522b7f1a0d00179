"""Per-kernel device time of the decode step's kernels at StarCoder2-3B layer sizes.

    python -m matricxon_b200.ops.microbench [rows]

Each kernel is captured 100 times in one CUDA graph (a dependent chain on one stream, hot
clocks) and the replay is timed with CUDA events: what the kernel costs inside a decode
graph, which a profiler's serialised, cold-clock launches overstate for small kernels.
"""
import sys

import torch

from matricxon_b200.ops import kernels as k
from matricxon_b200.ops.linear import linear


def main() -> None:
    dev = 'cuda:0'
    M = int(sys.argv[1]) if len(sys.argv) > 1 else 8
    H, I, NH, NKV, HD = 3072, 12288, 24, 2, 128
    QKV = (NH + 2 * NKV) * HD
    torch.manual_seed(0)
    x = torch.randn(M, H, device=dev)
    h = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
    g = torch.ones(H, device=dev); b = torch.zeros(H, device=dev)
    wqkv = torch.randn(QKV, H, device=dev).bfloat16() * 0.02
    wo = torch.randn(H, NH * HD, device=dev).bfloat16() * 0.02
    wfc = torch.randn(I, H, device=dev).bfloat16() * 0.02
    wpr = torch.randn(H, I, device=dev).bfloat16() * 0.02
    bq = torch.zeros(QKV, device=dev); bo = torch.zeros(H, device=dev); bfc = torch.zeros(I, device=dev)
    qkv = torch.empty(M, QKV, device=dev, dtype=torch.bfloat16)
    attn = torch.randn(M, NH * HD, device=dev).bfloat16()
    mid = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ctxlen = 3072; ps = 16; pages_per = ctxlen // ps + 1
    cache = torch.randn(M * pages_per, 2, NKV, ps, HD, device=dev).bfloat16()
    tables = torch.arange(M * pages_per, dtype=torch.int32, device=dev).view(M, pages_per).contiguous()
    positions = torch.full((M,), ctxlen, dtype=torch.int32, device=dev)
    slots = (tables[:, ctxlen // ps] * ps + ctxlen % ps).int().contiguous()
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, HD, 2, dtype=torch.float32) / HD))).to(dev)
    cu_q = torch.arange(M + 1, dtype=torch.int32, device=dev)
    ctx_lens = torch.full((M,), ctxlen, dtype=torch.int32, device=dev)
    narrow, wide = k.attention_tile_lists([1] * M, NH // NKV)
    tiles = torch.tensor(narrow, dtype=torch.int32, device=dev)
    n_splits = max(1, min(148 // (M * NKV), (ctxlen // 32 + 1) // 4, 128))
    scratch = torch.empty(k.attention_scratch_bytes(M, NH, HD, max(n_splits, 2)) // 4 + 16, device=dev)
    ops = {
        'layernorm': lambda: k.layernorm(x, g, b, 1e-5, h),
        'qkv skinny': lambda: k.gemm_skinny(h, wqkv, bq, None, qkv, 0),
        'rope_kv_write': lambda: k.rope_kv_write(qkv, positions, inv_freq, slots, cache, NH, NKV, HD, HD, ps, status),
        'qkv skinny + rotation + cache write (one kernel; not in the total)': lambda: k.gemm_skinny_rope(h, wqkv, bq, qkv, positions, inv_freq, slots, cache, NH, NKV, HD, ps, status),
        f'attention narrow (+merge) splits={n_splits}': lambda: k.paged_attention_mma(qkv, QKV, cache, tables, cu_q, ctx_lens, tiles, M, True, M, NH, NKV, HD, 4096, HD ** -0.5, attn, status, n_splits=n_splits, scratch=scratch),
        'o skinny residual': lambda: k.gemm_skinny(attn, wo, bo, x, x, 2),
        'c_fc skinny gelu': lambda: k.gemm_skinny(h, wfc, bfc, None, mid, 1),
        'c_proj skinny residual': lambda: k.gemm_skinny(mid, wpr, bo, x, x, 2),
    }
    if M > 16:
        del ops['qkv skinny + rotation + cache write (one kernel; not in the total)']
        ops['qkv skinny'] = lambda: linear(h, wqkv, bq, 0, out=qkv)
        ops['o skinny residual'] = lambda: linear(attn, wo, bo, 2, residual=x, out=x)
        ops['c_fc skinny gelu'] = lambda: linear(h, wfc, bfc, 1, out=mid)
        ops['c_proj skinny residual'] = lambda: linear(mid, wpr, bo, 2, residual=x, out=x)
    REP = 100
    total = 0.0
    for name, fn in ops.items():
        for _ in range(3): fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(REP): fn()
        graph.replay(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5): graph.replay()
        e1.record(); torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1000 / (5 * REP)
        if 'not in the total' not in name:
            total += us * (2 if name == 'layernorm' else 1)
        print(f"{name:45s} {us:8.2f} us")
    print(f"layer total (2 LN) {total:.1f} us  -> x30 = {total*30/1000:.2f} ms")


if __name__ == "__main__":
    main()

"""Device time of the prompt-attention kernels alone at StarCoder2-3B head geometry.

    python -m matricxon_b200.ops.attention_bench [tokens context [kernel [key_splits]]]

One sequence of ``tokens`` new tokens after ``context`` cached ones (24 query heads, 2 KV heads,
head_dim 128, pages of 16), the tcgen05 kernel ("tc") and the mma.sync kernel ("mma"), 20 launches
timed with CUDA events after 3 warm-up launches. Without arguments a few shapes are run.
"""
import sys

import torch

from matricxon_b200.ops import kernels as k
dev = "cuda:0"
H, KV, HD, ps = 24, 2, 128, 16
def run(n_tok, ctx, impl, splits=1):
    torch.manual_seed(0)
    total = ctx + n_tok
    pages = (total + ps - 1) // ps + 1
    qkv = torch.randn(n_tok, (H + 2 * KV) * HD, device=dev).bfloat16()
    cache = torch.randn(pages, 2, KV, ps, HD, device=dev).bfloat16()
    tables = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
    cu_q = torch.tensor([0, n_tok], dtype=torch.int32, device=dev)
    ctx_l = torch.tensor([ctx], dtype=torch.int32, device=dev)
    out = torch.empty(n_tok, H * HD, device=dev, dtype=torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    narrow, wide = k.attention_tile_lists([n_tok], H // KV, token_tiles=(impl == "tc"))
    tiles = torch.tensor(wide, dtype=torch.int32, device=dev)
    scratch = torch.empty(k.attention_scratch_bytes(n_tok, H, HD, splits) // 4 + 1, device=dev) if splits > 1 else None
    def call():
        if impl == "tc":
            k.paged_attention_tc(qkv, qkv.stride(0), cache, tables, cu_q, ctx_l, tiles, len(wide) // 2, n_tok, H, KV, HD, None, HD ** -0.5, out, st, n_splits=splits, scratch=scratch)
        else:
            k.paged_attention_mma(qkv, qkv.stride(0), cache, tables, cu_q, ctx_l, tiles, len(wide) // 2, False, n_tok, H, KV, HD, None, HD ** -0.5, out, st)
    for _ in range(3): call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20): call()
    e1.record(); torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 20
    flops = 4.0 * H * HD * (n_tok * ctx + n_tok * (n_tok + 1) / 2)
    print(f"{impl:4s} tokens {n_tok} ctx {ctx} splits {splits}: {us:8.1f} us  {flops / us / 1e6:7.1f} TFLOP/s  status {st.item()}")
if __name__ == "__main__":
    if len(sys.argv) >= 3:
        for impl in ([sys.argv[3]] if len(sys.argv) > 3 else ["mma", "tc"]):
            run(int(sys.argv[1]), int(sys.argv[2]), impl, int(sys.argv[4]) if len(sys.argv) > 4 else 1)
    else:
        for n_tok, ctx in ((2048, 0), (2048, 2048), (512, 3584), (256, 0)):
            for impl in ("mma", "tc"):
                run(n_tok, ctx, impl)

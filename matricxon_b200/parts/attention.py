"""Grouped-query attention over the paged cache.

``q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv`` (three Linear modules in the reference,
app/architectures/qwen_layers.py:50-52,71; packed here into one product), heads split as
feature ``head * head_dim + d`` (qwen_layers.py:72-74), position encoding on q and k
(qwen_layers.py:80), k and v stored (k already rotated, qwen_layers.py:83-86), scores scaled by
``scale`` with the causal rule ``j <= p`` (qwen_layers.py:12-17) and, when ``window`` is set,
``j > p - window`` (app/architectures/gemma4_layers.py:17-34, app/native/src/mx_attention.c:36-39);
query head h uses KV head ``h // (heads / kv heads)`` (qwen_layers.py:90-100); then
``residual + o Wo^T + bo`` (qwen_layers.py:101-102, app/architectures/starcoder2_layers.py:67).

Which kernel runs a step's rows, how the rows are cut into tiles and into how many pieces the
keys of a tile are split is decided here, beside the kernels' wrappers: the step context only
says what the step looks like (``host.q_lens``, ``max_kv_len``, ``sm_count``) and hands out
scratch memory (``ctx.scratch``) and a per-step memo (``ctx.memo``) so that layers with the same
geometry build their tile lists once.
"""

from __future__ import annotations

import os

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_NONE, EPILOGUE_RESIDUAL, chosen_backend, linear
from matricxon_b200.parts.base import KVCacheRequest, Mixer, build_part, register_part
from matricxon_b200.parts.rotary import store_without_rotation
from matricxon_b200.weights.loader import WeightSpec


# MATRICXON_TC_ATTENTION=0 keeps prompt portions on the mma.sync kernel (for comparisons)
_TC_ATTENTION = os.environ.get("MATRICXON_TC_ATTENTION", "1") != "0"


# ---------------------------------------------------------------------- tiling and key splits
def attention_tiles(ctx, group: int, token_tiles: bool = False):
    """Tile lists of the tensor-core attention for query groups of ``group`` heads:
    (narrow tiles, their count, wide tiles, their count); built once per step, group and
    kind of wide tile (64 rows, or ``token_tiles``: 128 // group tokens for the tcgen05 kernel)."""
    key = ("attention_tiles", group, token_tiles)
    cached = ctx.memo.get(key)
    if cached is not None:
        return cached
    q_lens = [1] * ctx.n_seqs if ctx.padded else ctx.host.q_lens
    narrow, wide = kernels.attention_tile_lists(q_lens, group, token_tiles)
    both = torch.tensor(narrow + wide + [0, 0], dtype=torch.int32).to(ctx.device, non_blocking=True)
    ctx.memo[key] = (both[:len(narrow)], len(narrow) // 2,
                     both[len(narrow):len(narrow) + len(wide)], len(wide) // 2)
    return ctx.memo[key]


def _key_span(ctx, window: int | None) -> int:
    return ctx.max_kv_len if window is None else min(ctx.max_kv_len, window)


def mma_tile_splits(ctx, n_tiles: int, narrow: bool, alone: bool, n_heads: int, n_kv_heads: int,
                    head_dim: int, window: int | None):
    """Key splits for one launch of the mma.sync attention (a block per tile, KV head and
    split). Splits only pay when the tiles alone leave SMs idle, and only a launch that covers
    every token of the step may use them (the merge runs over all tokens)."""
    if not alone:
        return 1, None
    items = max(n_tiles * n_kv_heads, 1)
    chunks = _key_span(ctx, window) // 32 + 1
    # a narrow block fills an SM's shared memory with its eight private stages: one per SM. A share of at
    # least eight chunks gives every warp of a narrow block one (a lone request at 3,100 tokens: 12 shares
    # of 8 chunks decode at 585 tok/s, 24 of 4 at 570, 48 of 2 at 520: more blocks, more to merge)
    target = ctx.sm_count * (1 if narrow else 2)
    n_splits = max(1, min(target // items, chunks // 8, 128))
    while n_splits > 1 and kernels.attention_scratch_bytes(
            ctx.n_tokens, n_heads, head_dim, n_splits) > (256 << 20):
        n_splits //= 2
    if n_splits == 1:
        return 1, None
    return n_splits, ctx.scratch(kernels.attention_scratch_bytes(ctx.n_tokens, n_heads, head_dim, n_splits))


def tc_tile_splits(ctx, n_tiles: int, alone: bool, n_heads: int, n_kv_heads: int, head_dim: int,
                   window: int | None):
    """Key splits for the tcgen05 attention (one block per SM, chunks of 128 keys): a short
    portion after a long context has few tiles with many chunks each."""
    items = max(n_tiles * n_kv_heads, 1)
    n_splits = min(ctx.sm_count // items, (_key_span(ctx, window) // 128 + 1) // 3, 8) if alone else 1
    if n_splits < 2:
        return 1, None
    return n_splits, ctx.scratch(kernels.attention_scratch_bytes(ctx.n_tokens, n_heads, head_dim, n_splits))


def simt_splits(ctx, n_heads: int, n_kv_heads: int, head_dim: int, window: int | None):
    """Key splits of the generic kernel: few query tokens (decoding) leave most SMs idle unless
    the keys are split; many tokens fill the GPU by themselves."""
    group = n_heads // n_kv_heads
    blocks = ctx.n_tokens * n_kv_heads * ((group + 15) // 16)
    chunks = _key_span(ctx, window) // 32 + 2
    n_splits = max(1, min(ctx.sm_count * 4 // max(blocks, 1), chunks // 2, 64))
    if n_splits == 1:
        return 1, None
    return n_splits, ctx.scratch(kernels.attention_scratch_bytes(ctx.n_tokens, n_heads, head_dim, n_splits))


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.position = (build_part("position", spec.position, runtime, prefix)
                         if spec.position is not None else None)
        # the kernels here are stream-ordered; a position encoding from elsewhere decides for itself
        self.capturable = self.position is None or self.position.capturable

    @classmethod
    def weight_specs(cls, spec, prefix):
        q_size, kv_size = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        if len(spec.projection_names) == 3:
            shapes = dict(zip(spec.projection_names, ((q_size, spec.hidden_size), (kv_size, spec.hidden_size),
                                                      (kv_size, spec.hidden_size))))
        else:
            shapes = {spec.projection_names[0]: (q_size + 2 * kv_size, spec.hidden_size)}
        shapes[spec.output_name] = (spec.hidden_size, q_size)
        specs = []
        for name, shape in shapes.items():
            specs.append(WeightSpec(f"{prefix}{name}.weight", shape, role="matrix", init="weight"))
            if spec.bias:
                specs.append(WeightSpec(f"{prefix}{name}.bias", (shape[0],), role="vector", init="bias"))
        return specs

    @classmethod
    def cache_request(cls, spec):
        return KVCacheRequest(num_kv_heads=spec.num_kv_heads, head_dim=spec.head_dim,
                              window=spec.window)

    def load(self, fetch):
        p, names = self.prefix, self.spec.projection_names

        def packed(kind: str) -> torch.Tensor:
            parts = [fetch(f"{p}{n}.{kind}") for n in names]
            return parts[0] if len(parts) == 1 else torch.cat(parts)

        self.qkv_weight = packed("weight")
        self.o_weight = fetch(f"{p}{self.spec.output_name}.weight")
        if self.spec.bias:
            self.qkv_bias = packed("bias")
            self.o_bias = fetch(f"{p}{self.spec.output_name}.bias")
        else:
            self.qkv_bias = self.o_bias = None

    def forward(self, h, residual, ctx, binding):
        spec, rt = self.spec, self.runtime
        if binding.kv is None:
            raise RuntimeError("attention needs cache pages bound to it")
        qkv = None
        if self.position is not None:
            qkv = self.position.project_rotate_store(h, self.qkv_weight, self.qkv_bias, ctx, binding,
                                                     spec.num_heads, spec.num_kv_heads, spec.head_dim)
        if qkv is not None:
            pass                                        # product, rotation and cache write were one kernel
        elif (self.position is not None and self.position.adds_bias and self.qkv_bias is not None
              and chosen_backend(h, self.qkv_weight, rt.gemm_backend) == "library"):
            # the library's product has no epilogue of its own: the rotation kernel adds the bias on its way
            qkv = linear(h, self.qkv_weight, None, EPILOGUE_NONE, backend=rt.gemm_backend)
            self.position.rotate_and_store(qkv, ctx, binding, spec.num_heads, spec.num_kv_heads,
                                           spec.head_dim, bias=self.qkv_bias)
        elif self.position is not None:
            qkv = linear(h, self.qkv_weight, self.qkv_bias, EPILOGUE_NONE, backend=rt.gemm_backend)
            self.position.rotate_and_store(qkv, ctx, binding, spec.num_heads, spec.num_kv_heads,
                                           spec.head_dim)
        else:
            qkv = linear(h, self.qkv_weight, self.qkv_bias, EPILOGUE_NONE, backend=rt.gemm_backend)
            store_without_rotation(qkv, ctx, binding, spec.num_heads, spec.num_kv_heads,
                                   spec.head_dim, rt.page_size)
        group = ctx.groups[binding.group]
        attn = torch.empty((ctx.n_tokens, self.q_size), dtype=rt.dtype, device=h.device)
        if kernels.mma_attention_supported(rt.dtype, spec.head_dim, rt.page_size, qkv.stride(0)):
            group_size = spec.num_heads // spec.num_kv_heads
            # prompt portions on tcgen05 when the kernel takes the geometry, else on mma.sync
            on_tc = _TC_ATTENTION and kernels.tc_attention_supported(rt.dtype, spec.head_dim, rt.page_size,
                                                                     qkv.stride(0), group_size)
            narrow, n_narrow, wide, n_wide = attention_tiles(ctx, group_size, token_tiles=on_tc)
            for tiles, n_tiles, is_narrow in ((narrow, n_narrow, True), (wide, n_wide, False)):
                if n_tiles == 0:
                    continue
                if on_tc and not is_narrow:
                    n_splits, scratch = tc_tile_splits(ctx, n_tiles, n_narrow == 0, spec.num_heads,
                                                           spec.num_kv_heads, spec.head_dim, spec.window)
                    kernels.paged_attention_tc(qkv, qkv.stride(0), binding.kv, group.block_tables, ctx.cu_q,
                                               ctx.context_lens, tiles, n_tiles, ctx.n_tokens,
                                               spec.num_heads, spec.num_kv_heads, spec.head_dim,
                                               spec.window, spec.scale, attn, ctx.status,
                                               n_splits=n_splits, scratch=scratch)
                    continue
                alone = (n_wide == 0) if is_narrow else (n_narrow == 0)
                if is_narrow and ctx.padded:
                    tiles, n_tiles = None, ctx.n_seqs      # a batch of decoding requests: tile i is sequence i
                n_splits, scratch = mma_tile_splits(ctx, n_tiles, is_narrow, alone, spec.num_heads,
                                                    spec.num_kv_heads, spec.head_dim, spec.window)
                kernels.paged_attention_mma(qkv, qkv.stride(0), binding.kv, group.block_tables,
                                            ctx.cu_q, ctx.context_lens, tiles, n_tiles, is_narrow,
                                            ctx.n_tokens, spec.num_heads, spec.num_kv_heads,
                                            spec.head_dim, spec.window, spec.scale, attn, ctx.status,
                                            n_splits=n_splits, scratch=scratch)
        else:
            n_splits, scratch = simt_splits(ctx, spec.num_heads, spec.num_kv_heads,
                                                     spec.head_dim, spec.window)
            kernels.paged_attention(qkv, qkv.stride(0), binding.kv, group.block_tables, ctx.tok_seq,
                                    ctx.positions, ctx.n_tokens, spec.num_heads, spec.num_kv_heads,
                                    spec.head_dim, spec.window, spec.scale, attn, ctx.status,
                                    n_splits=n_splits, scratch=scratch)
        return linear(attn, self.o_weight, self.o_bias, EPILOGUE_RESIDUAL, residual=residual,
                      out=residual, backend=rt.gemm_backend, defer_sum=getattr(ctx, "sums_may_pend", False))

"""Grouped-query attention over the paged cache.

``q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv`` (three Linear modules in the reference,
app/architectures/qwen_layers.py:50-52,71; packed here into one product), heads split as
feature ``head * head_dim + d`` (qwen_layers.py:72-74), position encoding on q and k
(qwen_layers.py:80), k and v stored (k already rotated, qwen_layers.py:83-86), scores scaled by
``scale`` with the causal rule ``j <= p`` (qwen_layers.py:12-17) and, when ``window`` is set,
``j > p - window`` (app/architectures/gemma4_layers.py:17-34, app/native/src/mx_attention.c:36-39);
query head h uses KV head ``h // (heads / kv heads)`` (qwen_layers.py:90-100); then
``residual + o Wo^T + bo`` (qwen_layers.py:101-102, app/architectures/starcoder2_layers.py:67).
"""

from __future__ import annotations

import os

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_NONE, EPILOGUE_RESIDUAL, linear
from matricxon_b200.parts.base import KVCacheRequest, Mixer, build_part, register_part
from matricxon_b200.parts.rotary import store_without_rotation
from matricxon_b200.weights.loader import WeightSpec


# MATRICXON_TC_ATTENTION=0 keeps prompt portions on the mma.sync kernel (for comparisons)
_TC_ATTENTION = os.environ.get("MATRICXON_TC_ATTENTION", "1") != "0"


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("attention heads must be a multiple of kv heads")
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.position = (build_part("position", spec.position, runtime, prefix)
                         if spec.position is not None else None)
        # the kernels here are stream-ordered; a position encoding from elsewhere decides for itself
        self.capturable = self.position is None or self.position.capturable

    @classmethod
    def weight_specs(cls, spec, prefix):
        q_size, kv_size = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        shapes = {"q_proj": (q_size, spec.hidden_size), "k_proj": (kv_size, spec.hidden_size),
                  "v_proj": (kv_size, spec.hidden_size), "o_proj": (spec.hidden_size, q_size)}
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
        p = self.prefix
        self.qkv_weight = torch.cat([fetch(f"{p}{n}.weight") for n in ("q_proj", "k_proj", "v_proj")])
        self.o_weight = fetch(f"{p}o_proj.weight")
        if self.spec.bias:
            self.qkv_bias = torch.cat([fetch(f"{p}{n}.bias") for n in ("q_proj", "k_proj", "v_proj")])
            self.o_bias = fetch(f"{p}o_proj.bias")
        else:
            self.qkv_bias = self.o_bias = None

    def describe(self):
        spec = self.spec
        return {"kind": "paged_attention", "qkv_weight": self.qkv_weight, "qkv_bias": self.qkv_bias,
                "o_weight": self.o_weight, "o_bias": self.o_bias, "num_heads": spec.num_heads,
                "num_kv_heads": spec.num_kv_heads, "head_dim": spec.head_dim, "window": spec.window,
                "scale": float(spec.scale),
                "position": self.position.describe() if self.position is not None else None}

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
            narrow, n_narrow, wide, n_wide = ctx.attention_tiles(group_size, token_tiles=on_tc)
            for tiles, n_tiles, is_narrow in ((narrow, n_narrow, True), (wide, n_wide, False)):
                if n_tiles == 0:
                    continue
                if on_tc and not is_narrow:
                    n_splits, scratch = ctx.tc_tile_splits(n_tiles, n_narrow == 0, spec.num_heads,
                                                           spec.num_kv_heads, spec.head_dim, spec.window)
                    kernels.paged_attention_tc(qkv, qkv.stride(0), binding.kv, group.block_tables, ctx.cu_q,
                                               ctx.context_lens, tiles, n_tiles, ctx.n_tokens,
                                               spec.num_heads, spec.num_kv_heads, spec.head_dim,
                                               spec.window, spec.scale, attn, ctx.status,
                                               n_splits=n_splits, scratch=scratch)
                    continue
                alone = (n_wide == 0) if is_narrow else (n_narrow == 0)
                n_splits, scratch = ctx.tile_splits(n_tiles, is_narrow, alone, spec.num_heads,
                                                    spec.num_kv_heads, spec.head_dim, spec.window)
                kernels.paged_attention_mma(qkv, qkv.stride(0), binding.kv, group.block_tables,
                                            ctx.cu_q, ctx.context_lens, tiles, n_tiles, is_narrow,
                                            ctx.n_tokens, spec.num_heads, spec.num_kv_heads,
                                            spec.head_dim, spec.window, spec.scale, attn, ctx.status,
                                            n_splits=n_splits, scratch=scratch)
        else:
            n_splits, scratch = ctx.attention_splits(spec.num_heads, spec.num_kv_heads,
                                                     spec.head_dim, spec.window)
            kernels.paged_attention(qkv, qkv.stride(0), binding.kv, group.block_tables, ctx.tok_seq,
                                    ctx.positions, ctx.n_tokens, spec.num_heads, spec.num_kv_heads,
                                    spec.head_dim, spec.window, spec.scale, attn, ctx.status,
                                    n_splits=n_splits, scratch=scratch)
        return linear(attn, self.o_weight, self.o_bias, EPILOGUE_RESIDUAL, residual=residual,
                      out=residual, backend=rt.gemm_backend)

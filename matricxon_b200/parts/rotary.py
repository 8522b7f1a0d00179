"""Rotary position encoding over whole heads, halves paired NeoX-style.

``inv_freq[i] = 1 / theta^(2i/dim)``; the angle of position p is ``p * inv_freq[i]``
in float32; ``o[i] = x[i] cos - x[i+dim/2] sin`` and ``o[i+dim/2] = x[i+dim/2] cos + x[i] sin``
(app/architectures/rope.py:16-29,152-169; app/native/src/mx_fused_ops.c:20-34). The
reference rounds cos and sin to the activation dtype before multiplying (rope.py:168);
here the rotation itself is float and the result is rounded once.

The table of inverse frequencies is built on the host exactly as the reference builds it,
so that angles at large positions agree to the last bit of the table.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.parts.base import PositionEncoding, register_part


def inverse_frequencies(rotary_dim: int, theta: float) -> torch.Tensor:
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
    return 1.0 / (theta ** exponent)


@register_part("position", "rotary_neox")
class RotaryNeox(PositionEncoding):
    capturable = True
    adds_bias = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.inv_freq = inverse_frequencies(spec.rotary_dim, spec.theta).to(runtime.device)

    def project_rotate_store(self, h, weight, bias, ctx, binding, n_heads, n_kv_heads, head_dim):
        rt = self.runtime
        if (rt.dtype != torch.bfloat16 or rt.gemm_backend != "auto" or self.spec.rotary_dim != head_dim
                or head_dim % 16 != 0 or not kernels.skinny_gemm_supported(h, weight)):
            return None
        writes = binding.writes and binding.kv is not None
        qkv = torch.empty((h.shape[0], weight.shape[0]), dtype=rt.dtype, device=h.device)
        kernels.gemm_skinny_rope(h, weight, bias, qkv, ctx.positions, self.inv_freq,
                                 ctx.groups[binding.group].slots if writes else None,
                                 binding.kv if writes else None, n_heads, n_kv_heads, head_dim,
                                 rt.page_size, ctx.status)
        return qkv

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim, bias=None):
        group = ctx.groups[binding.group] if binding.group is not None else None
        writes = binding.writes and binding.kv is not None
        kernels.rope_kv_write(
            qkv, ctx.positions, self.inv_freq,
            group.slots if writes else None, binding.kv if writes else None,
            n_heads, n_kv_heads, head_dim, self.spec.rotary_dim, self.runtime.page_size, ctx.status, bias=bias)


def store_without_rotation(qkv, ctx, binding, n_heads, n_kv_heads, head_dim, page_size):
    """Stores k and v as they are: what an attention layer without a position encoding needs,
    and what a position encoding written outside this package can call after its own rotation."""
    if not (binding.writes and binding.kv is not None):
        return
    empty = torch.empty(0, dtype=torch.float32, device=qkv.device)
    kernels.rope_kv_write(qkv, ctx.positions, empty, ctx.groups[binding.group].slots, binding.kv,
                          n_heads, n_kv_heads, head_dim, 0, page_size, ctx.status)

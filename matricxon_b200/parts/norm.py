"""LayerNorm with float statistics.

``(x - mean) / sqrt(var + eps) * weight + bias`` with the biased variance, as
nn.LayerNorm computes it in the reference (app/architectures/starcoder2_layers.py:45,56;
app/architectures/starcoder2.py:97). The input is the float32 residual stream; mean,
variance and the affine step stay float, and the result is rounded once to the runtime dtype.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.parts.base import Norm, register_part
from matricxon_b200.weights.loader import WeightSpec


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    capturable = True
    adds_pending_sum = True

    @classmethod
    def weight_specs(cls, spec, prefix):
        specs = [WeightSpec(prefix + "weight", (spec.size,), role="vector", init="norm_weight")]
        if spec.bias:
            specs.append(WeightSpec(prefix + "bias", (spec.size,), role="vector", init="norm_bias"))
        return specs

    def load(self, fetch):
        self.weight = fetch(self.prefix + "weight")
        self.bias = fetch(self.prefix + "bias") if self.spec.bias else None

    def forward(self, x, out=None, rows=None):
        n_rows = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n_rows, self.spec.size), dtype=self.runtime.dtype, device=x.device)
        kernels.layernorm(x, self.weight, self.bias, self.spec.eps, out, rows)
        return out

    def forward_sum(self, pending):
        """The norm of a residual sum that has not been added up yet (``ops.linear.PendingSum``): one
        kernel forms the sum, writes it to the residual stream and normalises it. Returns (x, norm(x))."""
        x = pending.added_by_kernel()
        out = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        kernels.layernorm_sum(x, pending.acc, pending.bias, self.weight, self.bias, self.spec.eps, out)
        return x, out

"""The plain (ungated) feed-forward: ``residual + down(act(up(h)))``.

``m = gelu_tanh(h Wfc^T + bfc)`` with ``gelu_tanh(u) = 0.5 u (1 + tanh(sqrt(2/pi)(u + 0.044715 u^3)))``,
then ``m Wproj^T + bproj`` added to the residual (app/architectures/starcoder2_layers.py:9-23,68).
The activation is applied to the float accumulator of the first product in the engine's own kernels;
for steps of 17 to 128 rows, where the library's product stands (ops/linear.py), to its bfloat16 result.
"""

from __future__ import annotations

from matricxon_b200.ops.linear import EPILOGUE_GELU, EPILOGUE_RESIDUAL, linear
from matricxon_b200.parts.base import FeedForward, register_part
from matricxon_b200.weights.loader import WeightSpec

_ACTIVATION_MODES = {"gelu_tanh": EPILOGUE_GELU}


@register_part("feed_forward", "mlp")
class Mlp(FeedForward):
    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        if spec.activation not in _ACTIVATION_MODES:
            raise ValueError(f"feed-forward activation {spec.activation!r} has no kernel")

    @classmethod
    def weight_specs(cls, spec, prefix):
        shapes = {spec.up_name: (spec.intermediate_size, spec.hidden_size),
                  spec.down_name: (spec.hidden_size, spec.intermediate_size)}
        specs = []
        for name, shape in shapes.items():
            specs.append(WeightSpec(f"{prefix}{name}.weight", shape, role="matrix", init="weight"))
            if spec.bias:
                specs.append(WeightSpec(f"{prefix}{name}.bias", (shape[0],), role="vector", init="bias"))
        return specs

    def load(self, fetch):
        p, s = self.prefix, self.spec
        self.up_weight = fetch(f"{p}{s.up_name}.weight")
        self.down_weight = fetch(f"{p}{s.down_name}.weight")
        self.up_bias = fetch(f"{p}{s.up_name}.bias") if s.bias else None
        self.down_bias = fetch(f"{p}{s.down_name}.bias") if s.bias else None

    def forward(self, h, residual, ctx):
        backend = self.runtime.gemm_backend
        mid = linear(h, self.up_weight, self.up_bias, _ACTIVATION_MODES[self.spec.activation],
                     backend=backend)
        return linear(mid, self.down_weight, self.down_bias, EPILOGUE_RESIDUAL, residual=residual,
                      out=residual, backend=backend, defer_sum=getattr(ctx, "sums_may_pend", False))

"""Arrangements of a mixer, a feed-forward and their norms inside one layer.

``pre_norm_sequential``: ``x = x + mixer(norm1(x)); x = x + ffn(norm2(x))``
(app/architectures/starcoder2_layers.py:67-68). The residual stream ``x`` is float32
and each sub-layer adds into it in float.
"""

from __future__ import annotations

from matricxon_b200.ops.linear import PendingSum
from matricxon_b200.parts.base import Block, build_part, register_part


@register_part("block", "pre_norm_sequential")
class PreNormSequentialBlock(Block):
    takes_pending_sum = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime, f"{prefix}{spec.mixer_norm_name}.")
        self.mixer = build_part("mixer", spec.mixer, runtime, f"{prefix}{spec.mixer_name}.")
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime, f"{prefix}{spec.ffn_norm_name}.")
        self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime,
                                       f"{prefix}{spec.feed_forward_name}.")
        self.capturable = all(part.capturable for part in self.parts())

    @classmethod
    def weight_specs(cls, spec, prefix):
        from matricxon_b200.parts.base import part_class

        out = []
        for category, sub, name in (("norm", spec.mixer_norm, spec.mixer_norm_name),
                                    ("mixer", spec.mixer, spec.mixer_name),
                                    ("norm", spec.ffn_norm, spec.ffn_norm_name),
                                    ("feed_forward", spec.feed_forward, spec.feed_forward_name)):
            out.extend(part_class(category, sub.kind).weight_specs(sub, f"{prefix}{name}."))
        return out

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    def load(self, fetch):
        for part in self.parts():
            part.load(fetch)

    @staticmethod
    def _normed(norm, x):
        """(x, norm(x)); ``x`` may arrive as a sum that the part before left to the norm to add up."""
        if isinstance(x, PendingSum):
            if norm.adds_pending_sum:
                return norm.forward_sum(x)
            x = x.tensor()
        return x, norm.forward(x)

    def forward(self, x, ctx, binding):
        """``x`` is the float residual stream or a ``PendingSum`` that stands for it; so is the result when
        the caller has said (``ctx.pending_sum_wanted``) that it takes one, else the result is the stream."""
        # this block knows what to do with a sum that one of its parts leaves pending; the parts only do so
        # on this say-so, which is withdrawn when the block is done
        ctx.sums_may_pend = True
        try:
            x, h = self._normed(self.mixer_norm, x)
            x = self.mixer.forward(h, x, ctx, binding)
            x, h = self._normed(self.ffn_norm, x)
            x = self.feed_forward.forward(h, x, ctx)
        finally:
            ctx.sums_may_pend = False
        if isinstance(x, PendingSum) and not getattr(ctx, "pending_sum_wanted", False):
            return x.tensor()
        return x

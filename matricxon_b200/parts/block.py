"""Arrangements of a mixer, a feed-forward and their norms inside one layer.

``pre_norm_sequential``: ``x = x + mixer(norm1(x)); x = x + ffn(norm2(x))``
(app/architectures/starcoder2_layers.py:67-68). The residual stream ``x`` is float32
and each sub-layer adds into it in float.
"""

from __future__ import annotations

from matricxon_b200.parts.base import Block, build_part, register_part


@register_part("block", "pre_norm_sequential")
class PreNormSequentialBlock(Block):
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

    def forward(self, x, ctx, binding):
        h = self.mixer_norm.forward(x)
        x = self.mixer.forward(h, x, ctx, binding)
        h = self.ffn_norm.forward(x)
        return self.feed_forward.forward(h, x, ctx)

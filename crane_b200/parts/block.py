"""Arrangements of parts in a layer.

``prenorm_residual``: h = norm1(x); x += mixer(h); h = norm2(x); x += ffn(h)
(crane-core/src/models/hunyuan_dense/modeling.rs:792-810).  Each addition is
fused into the norm that follows it, so a block hands its last output on
unadded ("pending") and receives the one of the block before it.
"""
from __future__ import annotations

from .base import build_part, register_block


@register_block("prenorm_residual")
class PreNormResidualBlock:
    """parts: ``norm1``, ``mixer``, ``norm2``, ``ffn``."""

    def __init__(self, layer_spec):
        self.norm1 = build_part(layer_spec.parts["norm1"])
        self.mixer = build_part(layer_spec.parts["mixer"])
        self.norm2 = build_part(layer_spec.parts["norm2"])
        self.ffn = build_part(layer_spec.parts["ffn"])

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def forward(self, x, pending, ctx, cache, rt):
        h = self.norm1.forward(x, pending, rt)
        a = self.mixer.forward(h, ctx, cache, rt)
        h = self.norm2.forward(x, a, rt)
        return self.ffn.forward(h, ctx, rt)

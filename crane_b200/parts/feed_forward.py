"""SiLU-gated feed-forward: down( silu(gate(h)) * up(h) ), no biases.

The gate and up matrices are merged into one [2I, H] product, as the reference
does (crane-core/src/models/hunyuan_dense/modeling.rs:667-694, 711-732);
silu(x) = x / (1 + exp(-x)) in 32-bit (crane-core/kernels/fused_ops.cu:39-42,
112-130).
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("ffn", "swiglu")
class SwiGLU(Part):
    """params: ``hidden_size``, ``intermediate_size``.  Tensors:
    ``<prefix>gate_proj.weight`` [I,H], ``up_proj.weight`` [I,H], ``down_proj.weight`` [H,I]."""
    kind = "ffn"

    @classmethod
    def manifest(cls, spec):
        h, i = spec.params["hidden_size"], spec.params["intermediate_size"]
        p = spec.prefix
        return {p + "gate_proj.weight": TensorSpec((i, h)), p + "up_proj.weight": TensorSpec((i, h)),
                p + "down_proj.weight": TensorSpec((h, i))}

    def load(self, weights, rt):
        p = self.prefix
        self.inter = int(self.params["intermediate_size"])
        self.gate_up = torch.cat([weights.pop(p + "gate_proj.weight"),
                                  weights.pop(p + "up_proj.weight")], dim=0).contiguous()
        self.down = weights[p + "down_proj.weight"]

    def forward(self, h, ctx, rt):
        gu = rt.linear(h, self.gate_up, None, "ffn_gate_up")
        act = rt.ws.get("ffn_act", h.shape[0], self.inter, rt.dtype)
        rt.kernels.silu_mul(gu, act)
        rt.launches += 1
        return rt.linear(act, self.down, None, "ffn_down")

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
        gate, up = weights.pop(p + "gate_proj.weight"), weights.pop(p + "up_proj.weight")
        # On the tensor-core path the merged matrix holds 16 gate rows, then the 16 up rows of
        # the same features, and so on: a tile of the product then has both halves of a
        # feature side by side and its epilogue can apply silu(gate) * up itself.
        self.blocked = (not rt.exact) and self.inter % 16 == 0
        if self.blocked:
            h = gate.shape[1]
            self.gate_up = torch.stack([gate.view(-1, 16, h), up.view(-1, 16, h)], dim=1).reshape(
                2 * self.inter, h).contiguous()
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.down = weights[p + "down_proj.weight"]

    def forward(self, h, ctx, rt):
        act = rt.ws.get("ffn_act", h.shape[0], self.inter, rt.dtype)
        if self.blocked and rt.linear_silu_mul(h, self.gate_up, act):
            return rt.linear(act, self.down, None, "ffn_down")
        gu = rt.linear(h, self.gate_up, None, "ffn_gate_up")
        rt.kernels.silu_mul(gu, act, self.blocked)
        rt.launches += 1
        return rt.linear(act, self.down, None, "ffn_down")

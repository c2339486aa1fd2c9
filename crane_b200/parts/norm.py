"""RMSNorm fused with the residual addition that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w, weight applied after normalising, sums in
32-bit (crane-core/kernels/fused_ops.cu:45-51, 183-232; the reference's fused
add+norm kernel exists but is never launched, fused_ops/cuda_impl.rs:241-260).
"""
from __future__ import annotations

from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("norm", "rms_norm")
class RMSNorm(Part):
    """params: ``size``, ``eps``.  Tensor: ``<prefix>weight`` [size], kept float."""
    kind = "norm"

    @classmethod
    def manifest(cls, spec):
        return {spec.prefix + "weight": TensorSpec((spec.params["size"],), "float32")}

    def load(self, weights, rt):
        self.weight = weights[self.prefix + "weight"]
        self.eps = float(self.params["eps"])
        self.size = int(self.params["size"])

    def forward(self, x, delta, rt, rows=None, name="normed"):
        """``x`` [N, size] float residual, updated in place by ``delta``;
        returns the normalised rows in the model dtype.  ``rows`` (int32 index
        tensor): normalise only x[rows] + delta[rows] and leave x alone."""
        n = x.shape[0] if rows is None else rows.shape[0]
        out = rt.ws.get(name, n, self.size, rt.dtype)
        rt.kernels.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        rt.launches += 1
        return out

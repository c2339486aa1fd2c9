"""Rotary position encoding with the base scaled by dynamic-NTK alpha.

inv_freq[j] = 1 / base^(2j/d), base = theta * alpha^(d/(d-2)) when alpha > 0;
the power in float64, rounded to float32, the reciprocal a float32 division;
angle[p, j] = float32(p) * inv_freq[j] as a float32 product; tables
[positions, d/2] of cos and sin in float32
(crane-core/src/models/hunyuan_dense/modeling.rs:197-239).  The reference
rounds the tables to the model dtype before use (modeling.rs:1004-1009); here
the angles stay 32-bit on every path.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Part, register_part

_TABLES = {}


@register_part("position", "rope")
class Rope(Part):
    """params: ``head_dim``, ``theta``, ``alpha`` (<= 0: none), ``max_positions``,
    ``rotary_dim`` (the rotated width of a head; default: all of it, which is
    what the reference does).  No tensors.  ``tables(rt, limit)`` gives (cos,
    sin) [positions < limit, rotary_dim / 2]."""
    kind = "position"

    def width(self) -> int:
        return int(self.params.get("rotary_dim") or self.params["head_dim"])

    def inv_freq(self) -> np.ndarray:
        d = self.width()
        base = float(self.params["theta"])
        alpha = float(self.params.get("alpha") or 0.0)
        if alpha > 0.0:
            # a head of 2 elements: the reference's float division gives an infinite exponent, the base
            # becomes infinite (or 0, or stays), and its power 0 is 1 either way
            base = base * alpha ** (d / (d - 2.0) if d != 2 else float("inf"))
        powers = np.array([base ** (i / d) for i in range(0, d, 2)], dtype=np.float64)
        return (np.float32(1.0) / powers.astype(np.float32)).astype(np.float32)

    def tables(self, rt, limit: int):
        n = min(int(self.params["max_positions"]), int(limit))
        key = (self.width(), float(self.params["theta"]),
               float(self.params.get("alpha") or 0.0), n, str(rt.device))
        if key not in _TABLES:
            pos = np.arange(n, dtype=np.float32)[:, None]
            angles = (pos * self.inv_freq()[None, :]).astype(np.float32)   # float32 product
            cos = np.cos(angles.astype(np.float64)).astype(np.float32)
            sin = np.sin(angles.astype(np.float64)).astype(np.float32)
            _TABLES[key] = (torch.from_numpy(cos).to(rt.device), torch.from_numpy(sin).to(rt.device))
        return _TABLES[key]

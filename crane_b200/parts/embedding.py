"""Token embedding and the output head.

x0 = E[token] without scaling (crane-core/src/models/hunyuan_dense/
modeling.rs:831-835, 998); logits = h W^T without bias, W the embedding table
when tied, else the top-level tensor ``lm_head.weight`` (modeling.rs:846-854).
Logits leave the head as float.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("embed", "token_embedding")
class TokenEmbedding(Part):
    """params: ``vocab_size``, ``hidden_size``.  Tensor: ``<prefix>weight`` [V,H]."""
    kind = "embed"

    @classmethod
    def manifest(cls, spec):
        return {spec.prefix + "weight": TensorSpec((spec.params["vocab_size"],
                                                    spec.params["hidden_size"]))}

    def load(self, weights, rt):
        self.table = weights[self.prefix + "weight"]

    def forward(self, tokens, x, rt, deferred=None):
        """Writes the float residual rows ``x`` [N,H] for int32 ``tokens`` [N].
        A token id <= -2 names row ``-id - 2`` of ``deferred`` (int32, on the
        device): a token sampled by an earlier launch that the host has not read."""
        rt.kernels.embed_gather(tokens, self.table, x, rt.err, deferred)
        rt.launches += 1


@register_part("head", "lm_head")
class LMHead(Part):
    """params: ``vocab_size``, ``hidden_size``, ``tied_to`` (name of the tensor
    it shares, or None).  Tensor when untied: ``<prefix>weight`` [V,H]."""
    kind = "head"

    @classmethod
    def manifest(cls, spec):
        if spec.params.get("tied_to"):
            return {}
        return {spec.prefix + "weight": TensorSpec((spec.params["vocab_size"],
                                                    spec.params["hidden_size"]))}

    def load(self, weights, rt):
        tied = self.params.get("tied_to")
        self.weight = weights[tied] if tied else weights[self.prefix + "weight"]

    def forward(self, h, rt):
        # wanted rows are few when serving; the buffer grows if a caller wants more
        return rt.linear(h, self.weight, None, "logits", out_dtype=torch.float32, cap=64)

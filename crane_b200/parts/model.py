"""A decoder put together from a ``ModelSpec``: embedding, blocks in the order
of the schedule, final norm over the wanted rows, head.

Nothing here names an architecture; the reference's counterpart is the
hard-wired ``HunYuanDenseV1`` (crane-core/src/models/hunyuan_dense/
modeling.rs:817-867, 990-1066).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.spec import ModelSpec
from ..weights.loader import TensorSpec, load_weights
from .base import CacheNeed, LayerCache, block_class, build_part, part_class


def _block_part_specs(layer_spec):
    return list(layer_spec.parts.values())


def model_manifest(spec: ModelSpec) -> Dict[str, TensorSpec]:
    """Every tensor the model expects, from the manifests of its parts."""
    out: Dict[str, TensorSpec] = {}
    specs = [spec.embed, spec.final_norm, spec.head]
    for layer in spec.layers:
        specs.extend(_block_part_specs(layer))
    for ps in specs:
        for name, ts in part_class(ps).manifest(ps).items():
            if name in out and out[name] != ts:
                raise ValueError(f"tensor {name} is claimed twice with different shapes")
            out[name] = ts
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, source, rt, where: str = "the model folder"):
        self.spec = spec
        self.rt = rt
        weights = load_weights(source, model_manifest(spec), spec.ignored_tensors, rt.dtype,
                               rt.device, where)
        self.embed = build_part(spec.embed)
        self.final_norm = build_part(spec.final_norm)
        self.head = build_part(spec.head)
        self.blocks = [block_class(l.block)(l) for l in spec.layers]
        # the head may share the embedding's tensor, so it loads before any part pops tensors
        self.embed.load(weights, rt)
        self.head.load(weights, rt)
        self.final_norm.load(weights, rt)
        for b in self.blocks:
            for part in b.parts():
                part.load(weights, rt)
        for place, step in enumerate(spec.schedule):
            if not 0 <= step.layer < len(self.blocks):
                raise ValueError(f"schedule step {place} names layer {step.layer}, which does not exist")
            src = step.cache_step(place)
            if not 0 <= src < len(spec.schedule) or spec.schedule[src].cache_of is not None and src != place:
                raise ValueError(f"schedule step {place} reads the cache of step {src}, "
                                 "which does not exist or has none of its own")

    def cache_needs(self) -> List[CacheNeed]:
        """Per step of the schedule, what its mixer keeps between engine steps
        (nothing for a step that reads another step's cache)."""
        return [self.blocks[s.layer].mixer.cache_need() if s.cache_of is None else CacheNeed("none")
                for s in self.spec.schedule]

    def capturable(self) -> bool:
        """Whether every part says that its forward can be recorded in a CUDA graph."""
        parts = [self.embed, self.final_norm, self.head]
        for b in self.blocks:
            parts += list(b.parts())
        return all(getattr(p, "capturable", True) for p in parts)

    def state_graph_safe(self) -> bool:
        """Whether every mixer that keeps per-request state bears graphs and padding."""
        return all(getattr(b.mixer, "state_graph_safe", False) for b in self.blocks
                   if b.mixer.cache_need().kind == "state")

    def forward(self, ctx, caches: List[LayerCache]) -> torch.Tensor:
        """Runs the step's tokens through the schedule (``caches``: one entry
        per step of the schedule) and returns float logits
        [wanted rows, vocab] (an empty tensor if nothing is wanted)."""
        rt = self.rt
        k = rt.kernels
        outer = k.pinned_stream
        k.pinned_stream = torch.cuda.current_stream(rt.device).cuda_stream
        try:
            return self._forward(ctx, caches)
        finally:
            k.pinned_stream = outer

    def _forward(self, ctx, caches: List[LayerCache]) -> torch.Tensor:
        rt = self.rt
        rt.begin_step()
        n = ctx.n_tokens
        x = rt.ws.get("residual", n, self.spec.hidden_size, torch.float32)
        self.embed.forward(ctx.tokens, x, rt, getattr(ctx, "deferred_tokens", None))
        pending = None
        for place, step in enumerate(self.spec.schedule):
            pending = self.blocks[step.layer].forward(x, pending, ctx, caches[step.cache_step(place)], rt)
        if ctx.n_want == 0:
            if pending is not None:
                pass   # the last block's output only feeds the head
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=rt.device)
        h = self.final_norm.forward(x, pending, rt, rows=ctx.want_rows, name="final_normed")
        return self.head.forward(h, rt)

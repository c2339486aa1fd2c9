"""What every part of a model is: a registered class that states the tensors it
expects, takes them, and runs on the rows it is given.

Interfaces (``rt`` is the ``Runtime``; ``ctx`` the ``StepContext`` of
``crane_b200.engine.step``):

* any part:     ``manifest(spec) -> {tensor name: TensorSpec}`` (class method),
                ``__init__(spec)``, ``load(weights, rt)``
* norm:         ``forward(x, delta, rt, rows=None) -> normed``; adds ``delta``
                into the float residual ``x`` in place, then normalises
* mixer:        ``cache_need() -> CacheNeed``; ``forward(h, ctx, cache, rt) -> Act``
* ffn:          ``forward(h, ctx, rt) -> Act``
* position:     ``tables(rt) -> (cos, sin)`` or whatever its mixer asks of it
* embed / head: ``forward(tokens, x, rt)`` / ``forward(h, rt) -> float logits``
* block:        ``forward(x, pending, ctx, cache, rt) -> pending``: takes the
                residual and the not-yet-added output of the block before it

An ``Act`` is a tensor [rows, cols] in the model dtype or ``Partials``.
A part never looks at the model it is in: all it knows is its ``spec.params``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple, Type

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorSpec

_PARTS: Dict[Tuple[str, str], Type["Part"]] = {}
_BLOCKS: Dict[str, Type] = {}


def register_part(kind: str, name: str) -> Callable[[Type["Part"]], Type["Part"]]:
    def deco(cls):
        _PARTS[(kind, name)] = cls
        return cls
    return deco


def register_block(name: str):
    def deco(cls):
        _BLOCKS[name] = cls
        return cls
    return deco


def part_class(spec: PartSpec) -> Type["Part"]:
    try:
        return _PARTS[(spec.kind, spec.name)]
    except KeyError:
        have = ", ".join(f"{k}:{n}" for k, n in sorted(_PARTS))
        raise KeyError(f"no {spec.kind} part named '{spec.name}' is registered; registered: {have}") from None


def build_part(spec: PartSpec) -> "Part":
    return part_class(spec)(spec)


def block_class(name: str):
    try:
        return _BLOCKS[name]
    except KeyError:
        raise KeyError(f"no block arrangement '{name}'; registered: {', '.join(sorted(_BLOCKS))}") from None


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps between steps, per request.
    ``kind == "kv"``: keys of ``kv_heads`` x ``head_dim`` and values of
    ``kv_heads`` x ``v_head_dim`` (0: as wide as the keys) per position in pages,
    all positions (``window == 0``) or the last ``window``.  The two pools are
    shaped independently, so values wider or narrower than keys need no change
    to the cache.
    ``kind == "state"``: one tensor of ``state_shape`` / ``state_dtype`` in the
    request's slot.  ``kind == "none"``: nothing (or another layer's cache)."""
    kind: str = "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: Tuple[int, ...] = ()
    state_dtype: torch.dtype = torch.float32
    v_head_dim: int = 0

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim


@dataclass
class LayerCache:
    """The storage one layer's mixer reads and writes.  For ``kv``: the K pool
    [pages, kv_heads, page_size, head_dim] and the V pool [pages, kv_heads,
    page_size, v_head_dim or head_dim] of the layer and the index of
    its layer group, whose block table for the step is
    ``ctx.block_tables[group]``.  For ``state``: a tensor [slots, *state_shape],
    indexed by ``ctx.slots``."""
    need: CacheNeed
    group: int = -1
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    page_size: int = 0
    state: Optional[torch.Tensor] = None


class Part:
    kind = "part"
    # Whether the part's forward can be recorded in a CUDA graph: it launches kernels and tensor
    # operations only and reads nothing of their results on the host.  A part that does read
    # (``.item()``, ``.cpu()``, ``nonzero()``, a data-dependent Python branch) sets this to False;
    # the engine then launches every step of the model kernel by kernel.
    capturable = True
    # For a mixer that keeps per-request state (``CacheNeed("state", ...)``): True says that it also
    # bears the padding of steps that replay graphs, which is what lets a model with such a mixer
    # replay graphs at all.  Its forward then reads the step's metadata on the device only (a graph
    # runs without the host), leaves rows whose ``tok_entry`` is -1 alone, and for an entry without
    # rows (``cu_q[e + 1] == cu_q[e]``, a padding entry) touches no slot, whatever ``slots[e]`` says.
    # Steps are only ever padded with such rows and entries, never with copies of an entry (a copy
    # would advance its request's state twice).
    state_graph_safe = False

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.params = spec.params
        self.prefix = spec.prefix

    @classmethod
    def manifest(cls, spec: PartSpec) -> Dict[str, TensorSpec]:
        return {}

    def load(self, weights: Dict[str, torch.Tensor], rt: "Runtime") -> None:
        pass


class Workspace:
    """Buffers that live as long as the engine, by name, sized for the largest
    step.  Their addresses never change, which is what replaying a captured
    graph needs."""

    def __init__(self, device, max_rows: int):
        self.device = device
        self.max_rows = max_rows
        self._bufs: Dict[Tuple[str, int, torch.dtype], torch.Tensor] = {}
        self._views: Dict[Tuple[str, int, int, torch.dtype], torch.Tensor] = {}
        self.generation = 0          # goes up whenever a buffer is replaced by a larger one

    def get(self, name: str, rows: int, cols: int, dtype: torch.dtype,
            cap: Optional[int] = None) -> torch.Tensor:
        """[rows, cols] of the buffer ``name``.  It is allocated for ``cap`` rows
        (default: the largest step) and only ever replaced by a larger one."""
        view = self._views.get((name, rows, cols, dtype))
        if view is not None:
            return view
        key = (name, cols, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[0] < rows:
            cap = max(rows, self.max_rows if cap is None else cap)
            if buf is not None:
                self.generation += 1
                self._views = {k: v for k, v in self._views.items() if (k[0], k[2], k[3]) != key}
            buf = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        view = buf[:rows]
        if len(self._views) < 4096:
            self._views[(name, rows, cols, dtype)] = view
        return view

    def zeros(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that starts as zeros and is never replaced (counters that
        kernels leave at zero)."""
        key = (name, cols, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[0] < rows:
            if buf is not None:
                self.generation += 1
                self._views = {k: v for k, v in self._views.items() if (k[0], k[2], k[3]) != key}
            buf = torch.zeros((rows, cols), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:rows]

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


def query_tiles(ctx, rows_per_tile: int, skip_single: bool = False) -> int:
    """How many tiles of ``rows_per_tile`` query rows the step's entries have, no
    tile spanning two entries (``skip_single``: not counting entries of exactly
    one token).  For a step that replays a captured graph (``ctx.graph_key``),
    the most that any step of the same shape can have: kernels skip the tiles
    beyond the real ones."""
    if getattr(ctx, "graph_key", None) is not None:
        return ctx.n_entries + ctx.n_tokens // rows_per_tile
    q_lens = ctx.h_cu_q[1:ctx.n_entries + 1] - ctx.h_cu_q[:ctx.n_entries]
    if skip_single:
        q_lens = q_lens[q_lens != 1]
    return int(((q_lens + rows_per_tile - 1) // rows_per_tile).sum())

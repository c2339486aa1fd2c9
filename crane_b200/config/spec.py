"""What a model is made of, as data: parts with their parameters, layer by layer,
and the order in which the layers run.

A configuration class turns its config.json into a ``ModelSpec``; nothing below
the spec knows which architecture it came from.  Every size and constant of a
part is in its ``params``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class PartSpec:
    """One part: ``kind`` is its role (mixer, ffn, norm, position, embed, head),
    ``name`` the registered implementation, ``params`` its sizes and constants,
    ``prefix`` the tensor-name prefix of its weights."""
    kind: str
    name: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass
class LayerSpec:
    """A block: which arrangement (``block``) of which parts."""
    block: str
    parts: Dict[str, PartSpec]


@dataclass
class ScheduleStep:
    """Run layer ``layer``.  Every step of the schedule has a cache of its own
    (so a layer that is named twice keeps two), unless ``cache_of`` names the
    step (by its place in the schedule) whose cache this one reads instead; a
    step that reads another's cache writes none."""
    layer: int
    cache_of: Optional[int] = None

    def cache_step(self, own_place: int) -> int:
        return own_place if self.cache_of is None else self.cache_of


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embed: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleStep]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: List[int] = field(default_factory=list)
    # tensors that a checkpoint of this architecture may hold and the model
    # never reads (name -> reason); they are not reported as unexpected
    ignored_tensors: Dict[str, str] = field(default_factory=dict)

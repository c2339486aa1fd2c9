"""From tensor names in a model folder to tensors on the device.

The parts of a model say which tensors they expect (name, shape, how it is
kept); ``load_weights`` compares that manifest with what the folder holds and
raises ONE error that lists every missing tensor, every unexpected tensor and
every wrong shape.  The reference leaves these errors to its tensor library
(crane-core/src/models/hunyuan_dense/model.rs:90-108).

How a tensor is kept:
* ``"model"``: in the engine's dtype: bfloat16 for serving, float32 on the
  true 32-bit path (the reference casts every tensor to the requested dtype
  on access, model.rs:90-94);
* ``"float32"``: always 32-bit (norm weights: norms are computed in 32-bit);
* ``"keep"``: as stored: a tensor stored in 32-bit stays so, integer tables
  become int32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Tuple

import torch

from .safetensors_io import TensorSource, model_files


class WeightsError(ValueError):
    """The folder's tensors do not match what the model expects."""

    def __init__(self, missing: List[str], unexpected: List[str],
                 wrong: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]], where: str):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"weights in {where} do not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + ", ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in wrong))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    keep: str = "model"        # "model" | "float32" | "keep"


def _target_dtype(spec: TensorSpec, stored: torch.dtype, model_dtype: torch.dtype) -> torch.dtype:
    if spec.keep == "float32":
        return torch.float32
    if spec.keep == "keep":
        if not stored.is_floating_point:
            return torch.int32
        return stored
    return model_dtype


def load_weights(source, manifest: Mapping[str, TensorSpec], ignored: Mapping[str, str],
                 model_dtype: torch.dtype, device, where: str = "the model folder"
                 ) -> Dict[str, torch.Tensor]:
    have = set(source.names())
    missing = sorted(n for n in manifest if n not in have)
    unexpected = sorted(n for n in have if n not in manifest and n not in ignored)
    wrong = []
    for n, spec in manifest.items():
        if n in have:
            _, shape = source.info(n)
            if tuple(shape) != tuple(spec.shape):
                wrong.append((n, tuple(spec.shape), tuple(shape)))
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, sorted(wrong), where)
    out: Dict[str, torch.Tensor] = {}
    for n, spec in manifest.items():
        t = source.tensor(n)
        out[n] = t.to(device=device, dtype=_target_dtype(spec, t.dtype, model_dtype)).contiguous()
    return out


def open_folder(folder: str) -> TensorSource:
    return TensorSource(model_files(folder))

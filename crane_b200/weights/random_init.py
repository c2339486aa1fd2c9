"""Random weights for a configuration and a seed, and the model folder
(config.json, model.safetensors) that holds them.

The reference has no such mode.  Matrices and biases are N(0, 0.02); tensors
that the model keeps in 32-bit (norm weights) are 1 + N(0, 0.01), so that no
norm is the identity.  Every tensor has its own generator, seeded from the
seed and the tensor's name, so the values do not depend on the order or on
which other tensors exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import torch

from ..config import resolve
from .loader import TensorSpec
from .safetensors_io import save_file


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensors(manifest: Dict[str, TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device="cpu", std: float = 0.02, norm_std: float = 0.01) -> Dict[str, torch.Tensor]:
    """One tensor per manifest entry.  ``dtype`` is how matrices are stored;
    32-bit tensors are always float32."""
    out: Dict[str, torch.Tensor] = {}
    dev = torch.device(device)
    for name in sorted(manifest):
        spec = manifest[name]
        gen = torch.Generator(device=dev)
        gen.manual_seed(_tensor_seed(seed, name))
        t = torch.randn(spec.shape, generator=gen, device=dev, dtype=torch.float32)
        is_norm_like = spec.keep == "float32" and name.endswith("weight")
        if is_norm_like:
            out[name] = (1.0 + norm_std * t)
        elif spec.keep == "float32":
            out[name] = std * t
        else:
            out[name] = (std * t).to(dtype)
    return out


def model_manifest_for(config: dict, model_type: Optional[str] = None):
    from ..parts import model_manifest
    arch = resolve(config, model_type)
    return model_manifest(arch.build_spec(arch.config_from_dict(config)))


def write_model_folder(folder: str, config: dict, seed: int, dtype: str = "bfloat16",
                       std: float = 0.02, norm_std: float = 0.01) -> str:
    """Writes ``config.json`` and ``model.safetensors`` with random weights of
    the architecture that ``config`` names.  ``dtype``: how matrices are stored
    ("bfloat16" or "float32")."""
    store = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
             "float32": torch.float32, "fp32": torch.float32}[dtype]
    os.makedirs(folder, exist_ok=True)
    tensors = random_tensors(model_manifest_for(config), seed, store, "cpu", std, norm_std)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"),
              {"format": "pt", "seed": seed, "generator": "crane_b200.weights.random_init"})
    return folder


def main(argv=None) -> int:
    """``python -m crane_b200.weights.random_init --config config.json --seed 0 --out DIR``"""
    import argparse
    ap = argparse.ArgumentParser(description="write a model folder with random weights")
    ap.add_argument("--config", required=True, help="a config.json of a registered architecture")
    ap.add_argument("--out", required=True, help="folder to write config.json and model.safetensors into")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="how matrices are stored")
    ap.add_argument("--std", type=float, default=0.02)
    args = ap.parse_args(argv)
    with open(args.config) as f:
        config = json.load(f)
    write_model_folder(args.out, config, args.seed, args.dtype, args.std)
    print(args.out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

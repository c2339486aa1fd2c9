"""Generation options, with the reference's names, defaults and meanings
(crane-core/src/generation/mod.rs:4-40)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class GenerationConfig:
    max_new_tokens: int = 245
    temperature: Optional[float] = 0.67     # None: greedy
    top_p: Optional[float] = 1.0
    repetition_penalty: float = 1.0         # != 1: applied to the last `repeat_last_n` tokens
    repeat_last_n: int = 5
    do_sample: bool = False                 # kept for parity; unused, as in the reference
    pad_token_id: Optional[int] = None      # unused, as in the reference
    eos_token_id: Optional[int] = None      # None: the model's (Hunyuan: 120020)
    report_speed: bool = False
    # beyond the reference's struct: its server's per-request options
    # (crane-serve/src/engine/types.rs:11-21)
    top_k: Optional[int] = None
    seed: Optional[int] = 1024              # the reference's fixed seed (hunyuan_dense/model.rs:304)

    @staticmethod
    def with_max_tokens(n: int) -> "GenerationConfig":
        return GenerationConfig(max_new_tokens=n)

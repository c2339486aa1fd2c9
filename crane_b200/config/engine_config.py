"""Settings of the engine that no config.json holds: precision, cache geometry,
batching limits.  Option names that the reference has keep its spelling and
meaning (crane-serve/src/lib.rs:27-52): ``max_concurrent``, ``max_seq_len``
(0: the model's limit), ``gpu_memory_limit``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPES = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32",
          "f32": "float32"}


def parse_memory_limit(text: Optional[str], total_bytes: int = 0) -> int:
    """"5G", "5120M", a fraction of the device's memory ("0.7") or bytes; 0 for
    none or for text that cannot be read (crane-serve/src/engine/mod.rs:94-129)."""
    if text is None:
        return 0
    s = text.strip()
    if not s or s == "0":
        return 0
    up = s.upper()
    for suffix, mult in (("G", 1 << 30), ("M", 1 << 20)):
        if up.endswith(suffix):
            try:
                return int(float(up[:-1].strip()) * mult)
            except ValueError:
                pass
    try:
        frac = float(s)
    except ValueError:
        return 0
    if 0.0 <= frac <= 1.0:
        return int(frac * total_bytes) if total_bytes > 0 else 0
    return int(frac) if frac > 1.0 else 0


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16": serving kernels; "float32": true 32-bit everywhere
    page_size: int = 64                # tokens per cache page
    num_pages: int = 0                 # pages per layer group; 0: from max_cache_tokens or memory
    max_cache_tokens: int = 0          # size the pool for this many tokens (rounded up to pages)
    gpu_memory_limit: Optional[str] = None
    max_concurrent: int = 16           # requests that hold cache at once
    max_seq_len: int = 0               # 0: max_position_embeddings
    max_batched_tokens: int = 2048     # token budget of one step
    chunk_size: int = 2048             # longest prompt portion of one request in a step
    workspace_rows: int = 0            # rows activations are first allocated for; 0: max_batched_tokens
    use_cuda_graphs: bool = True       # decode steps replay a captured graph (bfloat16 only)
    graph_max_tokens: int = 2048       # steps with prompt portions replay graphs too, up to this many tokens (0: never)
    async_scheduling: bool = True      # plan and launch a step before the last one's tokens are read
    mixed_decode_min_keys: int = 2048  # decoded tokens beside prompt portions take the split-KV decode
                                       # kernel when together they read at least this many cached keys
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {sorted(set(DTYPES))}, got {self.dtype!r}")
        self.dtype = DTYPES[self.dtype]
        if self.page_size <= 0 or self.page_size & (self.page_size - 1):
            raise ValueError(f"page_size must be a power of two, got {self.page_size}")
        if self.max_concurrent <= 0:
            raise ValueError("max_concurrent must be positive")
        if self.chunk_size <= 0 or self.max_batched_tokens <= 0:
            raise ValueError("chunk_size and max_batched_tokens must be positive")
        if self.max_batched_tokens < self.max_concurrent:
            raise ValueError(
                f"max_batched_tokens ({self.max_batched_tokens}) must be at least max_concurrent "
                f"({self.max_concurrent}) so that every running request can decode in a step")

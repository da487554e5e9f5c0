"""`EngineConfig`: the engine's own options, with the names and defaults of
tzar-beep/Tensorline's `BatchEngine` constructor and command line
(tensorline/batch_engine.py:79-85, tensorline/server.py:257-283)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class EngineConfig:
    dtype: str = "auto"                 # "auto" | "bfloat16" | "float32"; auto = bfloat16 on the GPU
    block_size: int = 16                # tokens per cache page
    num_blocks: int | None = None       # pages per group; None = from kv_cache_gb or free memory
    kv_mem_fraction: float = 0.6        # share of free device memory given to the cache when unsized
    kv_cache_gb: float | None = None
    max_num_seqs: int = 64
    max_batched_tokens: int = 2048
    max_model_len: int = 4096
    cuda_graphs: bool = True
    prefix_caching: bool = True
    graph_warmup_tokens: int = 512      # kept for the command line; graphs here do not depend on context length
    overlap: bool = True
    seed: int = 0

    def resolved_dtype(self, model_dtype: str | None = None) -> str:
        d = {"auto": None, "bf16": "bfloat16", "fp32": "float32", "float": "float32"}.get(self.dtype, self.dtype)
        if d is None:
            d = "bfloat16"
        if d not in ("bfloat16", "float32"):
            raise ValueError(f"dtype {self.dtype!r}: this engine runs 'bfloat16' or 'float32'")
        return d

    def validate(self) -> None:
        if self.block_size < 1 or self.block_size > 64 or 64 % self.block_size:
            raise ValueError(f"block_size {self.block_size}: must divide 64")
        if self.max_num_seqs < 1 or self.max_batched_tokens < 1 or self.max_model_len < 2:
            raise ValueError("max_num_seqs, max_batched_tokens and max_model_len must be positive")

"""Per-request sampling options and counters, with the fields and defaults of
tzar-beep/Tensorline's `SamplingParams` and `GenStats` (tensorline/engine.py:24-39)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 0.0            # <= 0 means greedy (tensorline/engine.py:43)
    top_p: float = 1.0
    stop_token_ids: set = field(default_factory=set)     # empty = the model's eos (batch_engine.py:176)
    seed: int | None = None             # None = engine seed mixed with the request id
    ignore_eos: bool = False            # never stop on a token; run to max_tokens


@dataclass
class GenStats:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0              # prompt tokens served from shared pages
    ttft_s: float = 0.0
    total_s: float = 0.0
    finish_reason: str = "length"

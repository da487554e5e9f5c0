"""The tiny configurations of the tests and helpers that write their model folders.

Tiny A and Tiny B differ in every size and option: layers, width, query heads, KV heads and group,
head size, feed-forward width (200 is no multiple of 64), vocabulary, rotary base, norm eps, tied or
untied head, norm weights, window (B: layers 1 and 2 see 24 keys), page size.
"""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tensorline_b200.config import Qwen2Config
from tensorline_b200.models import expected_tensors
from tensorline_b200.weights import write_random_model

TINY_A = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False,
              max_position_embeddings=4096, hidden_act="silu", eos_token_id=255)
TINY_B = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
              num_key_value_heads=1, head_dim=32, intermediate_size=200, vocab_size=384, rope_theta=1e6,
              rms_norm_eps=1e-5, tie_word_embeddings=False, use_sliding_window=True, sliding_window=24,
              max_window_layers=1, max_position_embeddings=2048, hidden_act="silu", eos_token_id=383)
# B without the window: for tests that need shared prefixes on an untied, group-3 model
TINY_B_FULL = dict(TINY_B, use_sliding_window=False)
# wider heads and a group of 7, as the large models have, still small
TINY_C = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=112, num_attention_heads=7,
              num_key_value_heads=1, head_dim=128, intermediate_size=304, vocab_size=500, rope_theta=1e6,
              rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
              max_position_embeddings=4096, hidden_act="silu", eos_token_id=499)

PAGE_SIZE = {"A": 4, "B": 8, "B_FULL": 8, "C": 16}
CONFIGS = {"A": TINY_A, "B": TINY_B, "B_FULL": TINY_B_FULL, "C": TINY_C}
# N(0, 0.02) as published checkpoints are initialised, and a wider draw that makes attention scores
# spread over several units so that a wrong key shows
INIT = {"A": dict(std=0.02, norm_std=0.0), "B": dict(std=0.08, norm_std=0.1),
        "B_FULL": dict(std=0.08, norm_std=0.1), "C": dict(std=0.05, norm_std=0.1)}


def write_tiny(name: str, folder=None, seed: int = 0, store_dtype=torch.bfloat16, **init) -> Path:
    cfg = Qwen2Config.from_dict(CONFIGS[name])
    folder = Path(folder) if folder is not None else Path(tempfile.mkdtemp(prefix=f"tiny_{name}_"))
    kw = dict(INIT[name])
    kw.update(init)
    return write_random_model(folder, cfg, expected_tensors(cfg), seed=seed, store_dtype=store_dtype, **kw)


def random_tokens(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

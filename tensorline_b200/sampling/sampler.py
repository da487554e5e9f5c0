"""Sampling one token per wanted row of logits, on the device.

Greedy rows take the argmax (tensorline/engine.py:43-44; batch_engine.py:386); others draw
from softmax(logits / temperature), cut to the top-p nucleus (tensorline/engine.py:45-50).
tzar-beep/Tensorline draws with the global generator (`torch.multinomial`, engine.py:51), so a
request's tokens depend on what else is running.  Here the uniform number of a draw is a hash of
(the request's seed, the index of the token being generated): the same request gives the same
tokens alone, in a batch, or recomputed after a preemption.
"""
from __future__ import annotations

import hashlib
import struct

import torch

from .. import ops
from .params import SamplingParams


def uniform_for(seed: int, token_index: int) -> float:
    """A float32-exact uniform in [0, 1) from (seed, token index)."""
    digest = hashlib.blake2b(struct.pack("<qq", seed & 0x7FFFFFFFFFFFFFFF, token_index), digest_size=8).digest()
    return (int.from_bytes(digest, "little") >> 40) / float(1 << 24)


def request_seed(engine_seed: int, rid: int, params: SamplingParams) -> int:
    if params.seed is not None:
        return int(params.seed)
    digest = hashlib.blake2b(struct.pack("<qq", engine_seed, rid), digest_size=8).digest()
    return int.from_bytes(digest, "little") & 0x7FFFFFFFFFFFFFFF


def draw_rows(rows: list):
    """`rows`: one (params, seed, token_index) each.  None if every row is greedy, else the numbers the
    sampling kernel needs, as three lists: temperatures, top-p values, uniform numbers."""
    if all(p.temperature <= 0 for p, _, _ in rows):
        return None
    return ([p.temperature for p, _, _ in rows], [p.top_p for p, _, _ in rows], [uniform_for(s, i) for _, s, i in rows])


class Sampler:
    def __init__(self, device):
        self.device = device

    @torch.inference_mode()
    def sample(self, logits: torch.Tensor, rows: list) -> list:
        """`rows`: one (params, seed, token_index) per row of `logits`.  Returns token ids."""
        R = logits.shape[0]
        if R == 0:
            return []
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        draw = draw_rows(rows)
        if draw is None:
            ops.argmax(logits, out)
        else:
            dev = torch.tensor(draw, dtype=torch.float32).to(logits.device)
            ops.sample(logits, dev[0], dev[1], dev[2], out)
        return out.tolist()

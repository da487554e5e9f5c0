"""Rotary position encoding, rotate-half pairing (tensorline/fused.py:34-51, :83-85).

tzar-beep/Tensorline takes the cos/sin table from an installed package
(tensorline/paged.py:241-242); the table here is the standard one: inv_freq[i] = theta^(-2i/rot),
i in [0, rot/2), held in float32; the angle pos * inv_freq[i] and its cosine and sine are
computed in float32 inside the kernel that also writes k and v to their pages.  `rotary_dim`
smaller than the head size leaves the remaining dimensions unrotated.
"""
from __future__ import annotations

import torch

from .base import Part, Rotary, Runtime, register_position_encoding


@register_position_encoding("rotary_half")
class RotaryHalf(Part):
    graph_capturable = True

    def __init__(self, rt: Runtime, head_dim: int, theta: float, rotary_dim: int | None = None):
        super().__init__(rt)
        rot = head_dim if rotary_dim is None else rotary_dim
        if rot % 2 or rot > head_dim or rot < 0:
            raise ValueError(f"rotary_dim {rot} must be even and at most head_dim {head_dim}")
        self.rot = rot
        i = torch.arange(0, rot, 2, dtype=torch.float64)
        self.inv_freq = (float(theta) ** (-i / rot)).to(torch.float32).to(rt.device)

    def rotary(self):
        return Rotary(self.inv_freq, self.rot, "half")

    def on_embedding(self, x, ctx):
        return None


@register_position_encoding("none")
class NoPositionEncoding(Part):
    graph_capturable = True

    def __init__(self, rt: Runtime, **_):
        super().__init__(rt)
        self._empty = torch.zeros(0, dtype=torch.float32, device=rt.device)

    def rotary(self):
        return Rotary(self._empty, 0)

    def on_embedding(self, x, ctx):
        return None

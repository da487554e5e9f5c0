"""Dense gated feed-forward: y = (act(h Wg^T) * (h Wu^T)) Wd^T, act = silu, no biases.

tzar-beep/Tensorline calls the installed package's module for this (tensorline/paged.py:276;
shapes tensorline/manager.py:53-54).  Here gate and up are one product against the stacked
[2I, H] matrix, the activation is a kernel of its own in float32, then the down product.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec, register_feed_forward
from .linear import matmul


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    def __init__(self, rt: Runtime, hidden: int, intermediate: int, activation: str = "silu"):
        super().__init__(rt)
        if activation != "silu":
            raise ValueError(f"gated_mlp runs 'silu', not {activation!r}")
        self.hidden, self.intermediate = hidden, intermediate
        self.w_gate_up = self.w_down = None

    def expected_tensors(self, prefix):
        H, I = self.hidden, self.intermediate
        return {f"{prefix}.gate_proj.weight": TensorSpec((I, H)), f"{prefix}.up_proj.weight": TensorSpec((I, H)),
                f"{prefix}.down_proj.weight": TensorSpec((H, I))}

    def bind(self, weights, prefix):
        g, u = weights[f"{prefix}.gate_proj.weight"], weights[f"{prefix}.up_proj.weight"]
        self.w_gate_up = self._compute_copy(torch.cat((g, u), dim=0))
        self.w_down = self._compute_copy(weights[f"{prefix}.down_proj.weight"])

    def forward(self, h, ctx):
        gu = matmul(h, self.w_gate_up)
        m = torch.empty((h.shape[0], self.intermediate), dtype=h.dtype, device=h.device)
        ops.silu_mul(gu, m)
        return matmul(m, self.w_down, may_defer=True)          # the next norm adds it up

"""Dense gated feed-forward: y = (act(h Wg^T) * (h Wu^T)) Wd^T, act = silu, no biases.

tzar-beep/Tensorline calls the installed package's module for this (tensorline/paged.py:276;
shapes tensorline/manager.py:53-54).  Here gate and up are one product against the stacked
[2I, H] matrix, the activation in float32 (the epilogue of the tcgen05 products for steps of few
tokens and for long steps, a kernel of its own in between), then the down product.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec, register_feed_forward
from .linear import NormedInput, matmul, use_pair_product, use_tc

GATE_BLOCK = 64


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    graph_capturable = True
    accepts_normed_input = True         # `h` may be a `NormedInput`: the gate|up product normalises it on the fly

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
        I, H = self.intermediate, self.hidden
        # bfloat16 engine, I % 64 == 0: gate and up rows alternate in blocks of 64, so that a 128-row tile of
        # the tcgen05 product holds both halves of 64 output columns and its epilogue can apply the activation
        self.block = GATE_BLOCK if (self.rt.act_dtype == torch.bfloat16 and I % GATE_BLOCK == 0) else None
        if self.block:
            gu = torch.stack((g.view(I // GATE_BLOCK, GATE_BLOCK, H), u.view(I // GATE_BLOCK, GATE_BLOCK, H)), dim=1)
            self.w_gate_up = self._compute_copy(gu.reshape(2 * I, H))
        else:
            self.w_gate_up = self._compute_copy(torch.cat((g, u), dim=0))
        self.w_down = self._compute_copy(weights[f"{prefix}.down_proj.weight"])

    def forward(self, h, ctx):
        I = self.intermediate
        if isinstance(h, NormedInput) and h.rows is not None:
            h = h.materialize()
        if self.block and h.dtype == torch.bfloat16 and h.is_contiguous() and use_tc(h.shape[0], 2 * I, self.hidden):
            from .. import ops_gemm
            if ops_gemm.can_gate(h.shape[0], 2 * I, self.hidden):          # the activation inside the product
                m = ops_gemm.gemm_tc(h, self.w_gate_up, gated=True)
                return matmul(m, self.w_down, may_defer=True, to_residual=True)
        if isinstance(h, NormedInput):                   # only the few-token products above take the recipe
            h = h.materialize()
        if self.block and h.dtype == torch.bfloat16 and h.is_contiguous() and use_pair_product(h.shape[0], 2 * I, self.hidden):
            from .. import ops_gemm
            m = ops_gemm.gemm_tc2(h, self.w_gate_up, gated=True)          # long steps: pairs of blocks, activation in the epilogue
            return matmul(m, self.w_down, may_defer=True)
        gu = matmul(h, self.w_gate_up)
        m = torch.empty((h.shape[0], I), dtype=h.dtype, device=h.device)
        ops.silu_mul(gu, m, block=self.block)
        return matmul(m, self.w_down, may_defer=True, to_residual=True)          # the next norm adds it up

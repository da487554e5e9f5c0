"""RMSNorm with the residual add folded in (tensorline/fused.py:19-32, :58-69)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec, register_norm
from .linear import FUSE_NORMS, NormedInput, PendingProduct, SplitSum


@register_norm("rms_norm")
class RMSNorm(Part):
    graph_capturable = True
    can_defer = True                    # add_norm(..., defer=True) may return a `NormedInput`

    def __init__(self, rt: Runtime, dim: int, eps: float):
        super().__init__(rt)
        self.dim, self.eps = dim, eps
        self.weight = None

    def expected_tensors(self, prefix):
        return {f"{prefix}.weight": TensorSpec((self.dim,), init="ones")}

    def bind(self, weights, prefix):
        self.weight = weights[f"{prefix}.weight"].contiguous()      # stays in its stored type

    def add_norm(self, x, pending, rows=None, defer=False):
        """`defer`: the caller's next step is a product that takes a `NormedInput`."""
        n = x.shape[0] if rows is None else rows.numel()
        if isinstance(pending, PendingProduct):
            ssq = pending.add_into(x)                    # the product adds its result into x itself, where its plan allows
            if ssq is None:
                pending = pending.run()
            else:                                        # x holds the sum (also with `rows`: nobody reads x after the last norm)
                if defer and FUSE_NORMS and self.dim % 8 == 0 and self.weight.dtype in (torch.float32, torch.bfloat16):
                    return NormedInput(x, ssq, self.weight, self.eps, rows, self.rt.act_dtype)
                h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
                ops.add_rmsnorm(x, None, self.weight, h, self.eps, rows=rows)
                return h
        h = torch.empty((n, self.dim), dtype=self.rt.act_dtype, device=x.device)
        if isinstance(pending, SplitSum):                # a split-K product: its pieces are summed inside the kernel
            if pending.dtype == h.dtype and self.dim % 4 == 0 and self.dim <= 32768:
                ops.add_rmsnorm(x, None, self.weight, h, self.eps, rows=rows, pieces=pending.pieces)
                return h
            pending = pending.sum()
        ops.add_rmsnorm(x, pending, self.weight, h, self.eps, rows=rows)
        return h

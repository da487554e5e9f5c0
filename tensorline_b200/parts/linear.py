"""Matrix products of the parts: y = x W^T, weights [out, in] (tensorline/quant.py:3).

The 32-bit engine uses the exact-order FFMA kernel of this package.  The bfloat16 engine calls
the library product (cuBLAS through torch), as tzar-beep/Tensorline's engine does for every
projection (tensorline/paged.py:248-250, :275-276, :287), with float32 accumulation.
"""
from __future__ import annotations

import torch

from .. import ops


def matmul(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [T, K] (float32 or bfloat16) times w [N, K]^T -> [T, N]."""
    if x.dtype == torch.float32:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        ops.gemm_f32(x, w, out)
        return out
    if not x.is_cuda:
        raise ops.KernelError("matmul called with a CPU tensor: this engine has no CPU path")
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    return torch.mm(x, w.t())

"""Matrix products of the parts: y = x W^T, weights [out, in] (tensorline/quant.py:3).

The 32-bit engine uses the exact-order FFMA kernel of this package.  The bfloat16 engine has two
routes, both with float32 accumulation:
  * the hand-written tcgen05 / TMA kernel (`csrc/gemm_tc.cu`) for steps of few tokens against large
    matrices, where it streams the weights faster than the library and chains with the kernels around
    it (measured on the 7B shapes: every projection and the output head at up to 64 tokens);
  * the library product (cuBLAS through torch) everywhere else, as tzar-beep/Tensorline's engine does
    for every projection (tensorline/paged.py:248-250, :275-276, :287).
"""
from __future__ import annotations

import os

import torch

from .. import ops

TC_MAX_TOKENS = int(os.environ.get("TENSORLINE_B200_TC_MAX_TOKENS", 64))     # the hand-written kernel wins up to this many tokens ...
TC_MIN_WEIGHT_ELEMENTS = int(os.environ.get("TENSORLINE_B200_TC_MIN_ELEMENTS", 8 << 20))   # ... against matrices of at least this many elements


TC_ENABLED = os.environ.get("TENSORLINE_B200_TC", "1") != "0"   # 0: library products only (for A/B timing)


def use_tc(tokens: int, n: int, k: int) -> bool:
    return TC_ENABLED and tokens <= TC_MAX_TOKENS and n * k >= TC_MIN_WEIGHT_ELEMENTS and k % 8 == 0


# The two-block (cta_group::2) product with the activation in its epilogue takes the gate|up product of long steps.
# Measured against the library product followed by the activation kernel at the 7B / 14B / 32B shapes: 0.997 / 0.98 /
# 1.01 at 512 tokens, 1.02 / 0.99 / 1.00 at 1,024, 1.03 / 1.05 / 1.08 at 1,536, 1.04 / 1.02 / 1.07 at 2,048, 1.08 /
# 1.05 / 1.11 at 4,096; it works on tiles of 256 tokens, so a step that fills its last tile badly stays with the library.
PAIR_ENABLED = os.environ.get("TENSORLINE_B200_TC_PAIR_PRODUCT", "1") != "0"
PAIR_MIN_TOKENS = int(os.environ.get("TENSORLINE_B200_TC_PAIR_MIN_TOKENS", 1280))
PAIR_MAX_WASTE = 1.10


def use_pair_product(tokens: int, n: int, k: int) -> bool:
    return (TC_ENABLED and PAIR_ENABLED and tokens >= PAIR_MIN_TOKENS and -(-tokens // 256) * 256 <= PAIR_MAX_WASTE * tokens
            and n * k >= TC_MIN_WEIGHT_ELEMENTS and k % 8 == 0)


class SplitSum:
    """A product whose split-K pieces [S, T, N] (float32) have not been added up yet.  A consumer that
    reads its input once anyway (the residual add + norm) sums them on the way and saves the pass that
    would; anyone else calls `resolve`."""

    def __init__(self, pieces: torch.Tensor, dtype: torch.dtype):
        self.pieces, self.dtype = pieces, dtype
        self.shape = pieces.shape[1:]

    def sum(self) -> torch.Tensor:
        from .. import ops_gemm
        return ops_gemm.sum_pieces(self.pieces, self.dtype)


def resolve(t):
    """A tensor from what a projection returned."""
    return t.sum() if isinstance(t, SplitSum) else t


def matmul(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None, may_defer: bool = False):
    """x [T, K] (float32 or bfloat16) times w [N, K]^T -> [T, N].  `may_defer`: the caller hands the
    result to a consumer that takes a `SplitSum`."""
    if x.dtype == torch.float32:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        ops.gemm_f32(x, w, out)
        return out
    if not x.is_cuda:
        raise ops.KernelError("matmul called with a CPU tensor: this engine has no CPU path")
    if use_tc(x.shape[0], w.shape[0], w.shape[1]) and x.is_contiguous():
        from .. import ops_gemm
        y = ops_gemm.gemm_tc(x, w, out_dtype or x.dtype, pieces=may_defer)
        return SplitSum(y, out_dtype or x.dtype) if y.dim() == 3 else y
    y = torch.mm(x, w.t(), out_dtype=out_dtype) if out_dtype is not None and out_dtype != x.dtype else torch.mm(x, w.t())
    ops.mark("library product")
    return y

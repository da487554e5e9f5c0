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


# The layer's norms folded into the products around them (steps of few tokens, bfloat16): the product that makes an
# addend adds it into the residual stream in its own epilogue, and the product that reads a norm's result normalises its
# operand on the fly.  The norm kernel between them, which moves almost no bytes but costs a launch and two memory round
# trips, goes away (two a layer).  TENSORLINE_B200_FUSE_NORMS=0: every norm a kernel of its own (A/B timing).
FUSE_NORMS = os.environ.get("TENSORLINE_B200_FUSE_NORMS", "1") != "0"
# Every block of the reading product normalises the activations of its K range itself; with many tokens that is more
# traffic through L2 than the norm kernel saves, so steps of more tokens keep the norm kernel.
FUSE_NORMS_MAX_TOKENS = int(os.environ.get("TENSORLINE_B200_FUSE_NORMS_MAX_TOKENS", 16))


class PendingProduct:
    """A product x W^T that has not run yet and whose result is an addend of the residual stream.  Whoever adds it up
    (a norm) either lets the product do the addition itself (`add_into`) or runs it (`run`) and adds the result."""

    def __init__(self, x: torch.Tensor, w: torch.Tensor):
        self.x, self.w = x, w
        self.dtype, self.shape = x.dtype, (x.shape[0], w.shape[0])

    def run(self):
        """The product as a tensor, or as a `SplitSum`."""
        return matmul(self.x, self.w, may_defer=True)

    def add_into(self, stream: torch.Tensor):
        """stream += x W^T (rounded to the activation type first) inside the product's kernel; returns the partial sums
        of squares of the stream's new rows, float32 [T, parts], or None if these sizes do not take that path."""
        from .. import ops_gemm
        T, N, K = self.x.shape[0], self.w.shape[0], self.w.shape[1]
        if not (stream.dtype == torch.float32 and stream.shape == (T, N) and stream.is_contiguous() and N % 4 == 0
                and ops_gemm.can_add_residual(T, N, K)):
            return None
        return ops_gemm.gemm_tc(self.x, self.w, residual=stream)


class NormedInput:
    """Activations that exist only as their recipe: rows of the float32 residual stream `x`, the partial sums of squares
    of those rows `ssq` [rows of x, parts], the norm's weight and eps.  A product that takes it (`matmul`) normalises its
    operand inside its kernel; anyone else calls `materialize()`.  `rows`: int32 indices into x, or None for all rows."""

    def __init__(self, x, ssq, weight, eps, rows, dtype):
        self.x, self.ssq, self.weight, self.eps, self.rows, self.dtype = x, ssq, weight, eps, rows, dtype
        self.shape = (x.shape[0] if rows is None else rows.numel(), x.shape[1])
        self.device = x.device

    def is_contiguous(self) -> bool:
        return True

    def materialize(self) -> torch.Tensor:
        h = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        ops.add_rmsnorm(self.x, None, self.weight, h, self.eps, rows=self.rows)
        return h


def resolve(t):
    """A tensor from what a projection or a norm returned."""
    if isinstance(t, PendingProduct):
        t = t.run()
    if isinstance(t, NormedInput):
        return t.materialize()
    return t.sum() if isinstance(t, SplitSum) else t


def matmul(x, w: torch.Tensor, out_dtype: torch.dtype | None = None, may_defer: bool = False, to_residual: bool = False):
    """x [T, K] (float32 or bfloat16) times w [N, K]^T -> [T, N].  `may_defer`: the caller hands the
    result to a consumer that takes a `SplitSum`.  `to_residual`: the result is an addend of the residual stream and
    goes to a norm's `add_norm`: a `PendingProduct` may come back instead of a result.  `x` may be a `NormedInput`."""
    if isinstance(x, NormedInput):
        if x.rows is None and use_tc(x.shape[0], w.shape[0], w.shape[1]) and w.dtype == torch.bfloat16:
            from .. import ops_gemm
            y = ops_gemm.gemm_tc(x, w, out_dtype or x.dtype, pieces=may_defer)
            return SplitSum(y, out_dtype or x.dtype) if y.dim() == 3 else y
        x = x.materialize()
    if to_residual and FUSE_NORMS and x.shape[0] <= FUSE_NORMS_MAX_TOKENS and x.dtype == torch.bfloat16 and x.is_cuda and \
            x.is_contiguous() and use_tc(x.shape[0], w.shape[0], w.shape[1]) and out_dtype in (None, x.dtype):
        return PendingProduct(x, w)
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

"""Launcher of the tcgen05 / TMA matrix product (`csrc/gemm_tc.cu`).

    y[T, N] = x[T, K] w[N, K]^T     bfloat16 in, float32 accumulation in tensor memory

With few tokens the weight matrix takes the 128-row side of the MMA tile ("swap") and, if it gives
fewer tiles than the GPU has SMs, the reduction is split across blocks.  A wait that runs out inside a
kernel is recorded in the device status word (`ops.device_status`), which the engine reads with every
step's tokens.  With `fused_reduce` the last block of a tile sums the
split partials inside the same launch instead of a second kernel (faster for one token, slower from a few
tokens on, so it is off by default).
"""
from __future__ import annotations

import ctypes
import os

import torch

from .csrc.build import load_library
from . import ops
from .ops import KernelError, _check, _ptr, _stream

_P, _I = ctypes.c_void_p, ctypes.c_int
_lib = None


def lib():
    global _lib
    if _lib is None:
        l = load_library("tl_gemm_tc", ["gemm_tc.cu"])
        l.tl_gemm_tc.argtypes = [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _I, _P]
        l.tl_gemm_tc.restype = ctypes.c_int
        l.tl_gemm_tc_normed.argtypes = [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _I,
                                        _P, _I, _P, _P, _P, _I, _P, _I, ctypes.c_float, _P]
        l.tl_gemm_tc_normed.restype = ctypes.c_int
        l.tl_splitk_reduce.argtypes = [_P, _P, _I, _I, _I, _I, _I, _P]
        l.tl_splitk_reduce.restype = ctypes.c_int
        _lib = l
    return _lib


N_COUNTERS = ops.N_COUNTERS
CLUSTER_MAX = 8                # portable cluster size
CLUSTER_REDUCE = os.environ.get("TENSORLINE_B200_CLUSTER_REDUCE", "1") != "0"   # 0: pieces + a summing pass (A/B timing)
status_word = ops.device_status
check_status = ops.check_device_status


def plan(T: int, N: int, K: int, sms: int | None = None) -> tuple:
    """(swap, bn, splits) for a product of T tokens on a GPU of `sms` multiprocessors."""
    NUM_SMS = sms or ops.num_sms()
    k_tiles = -(-K // 64)
    if T <= 64:
        bn = 16 if T <= 16 else 32 if T <= 32 else 64
        tiles = -(-N // 128)
        splits = 1
        if tiles < NUM_SMS:                           # too few tiles to give every SM a block: split K so that
            splits = max(1, min(k_tiles // 4, (2 * NUM_SMS - 40) // tiles))   # one round of blocks is nearly full
            if CLUSTER_REDUCE and splits > CLUSTER_MAX:
                splits = CLUSTER_MAX                  # the ranges of a tile then sum inside a thread-block cluster
        return 1, bn, splits
    return 0, 128 if N <= 4096 else 256, 1


def can_add_residual(T: int, N: int, K: int) -> bool:
    """Whether the plan for these sizes lets the product add its result into the residual stream itself: the few-token
    order with 2..8 K ranges summed inside a cluster."""
    swap, _, splits = plan(T, N, K)
    k_tiles = -(-K // 64)
    splits = -(-k_tiles // -(-k_tiles // min(splits, k_tiles)))
    return bool(swap) and CLUSTER_REDUCE and 2 <= splits <= CLUSTER_MAX and N % 4 == 0


def gemm_tc(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, *, swap=None, bn=None,
            splits=None, out: torch.Tensor | None = None, fused_reduce: bool = False, pieces: bool = False,
            gated: bool = False, cluster: bool | None = None, residual: torch.Tensor | None = None):
    """x [T, K] times w [N, K]^T.  With 2..8 K ranges (few-token order) the ranges of a tile form a
    thread-block cluster and sum through distributed shared memory (`cluster`; None = wherever it
    applies).  `pieces`: when K is split otherwise, return the float32 pieces [S, T, N] unsummed (for a
    consumer that adds them up itself) instead of the product.
    `gated`: w holds gate and up rows interleaved in blocks of 64 (N % 128 == 0); the result is
    silu(gate) * up, [T, N / 2] bfloat16, formed in the epilogue (few tokens, one split only:
    check `can_gate` first).
    `x` may be a `parts.linear.NormedInput` (few-token order): the activations are then the RMS norm of rows of the
    float32 residual stream, made inside the kernel from the stream, the rows' partial sums of squares and the norm weight.
    `residual` (float32 [T, N], check `can_add_residual` first): the result, rounded to bfloat16, is added into it in
    place inside the kernel; returned are the partial sums of squares of its new rows, float32 [T, ceil(N / 128)]."""
    normed = None
    if not isinstance(x, torch.Tensor):
        normed, x = x, None
        T, K = normed.shape
        if normed.rows is not None:
            raise KernelError("gemm_tc: a normed input that picks rows has to be materialized first")
        if normed.x.dtype != torch.float32 or not normed.x.is_contiguous() or normed.x.shape[1] != K or K % 8:
            raise KernelError("gemm_tc: a normed input needs a contiguous float32 stream of a width that is a multiple of 8")
        if normed.ssq.dtype != torch.float32 or not normed.ssq.is_contiguous() or normed.ssq.shape[0] != normed.x.shape[0]:
            raise KernelError("gemm_tc: a normed input needs float32 sums of squares, one row per row of the stream")
        if normed.weight.numel() != K or normed.weight.dtype not in (torch.float32, torch.bfloat16) or not normed.weight.is_contiguous():
            raise KernelError("gemm_tc: the norm weight must be float32 or bfloat16 [K]")
        dev = normed.x.device
    else:
        if x.dtype != torch.bfloat16:
            raise KernelError("gemm_tc: bfloat16 operands only")
        T, K = x.shape
        dev = x.device
    if w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: bfloat16 operands only")
    N = w.shape[0]
    if w.shape[1] != K or (x is not None and not x.is_contiguous()) or not w.is_contiguous():
        raise KernelError("gemm_tc: x [T, K] and w [N, K] must be contiguous with equal K")
    if K % 8:
        raise KernelError(f"gemm_tc: K = {K} must be a multiple of 8 (TMA needs 16-byte rows)")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tc: output is bfloat16 or float32")
    p_swap, p_bn, p_splits = plan(T, N, K)
    swap = p_swap if swap is None else int(swap)
    bn = p_bn if bn is None else bn
    splits = p_splits if splits is None else splits
    k_tiles = -(-K // 64)
    splits = -(-k_tiles // -(-k_tiles // min(splits, k_tiles)))          # as the kernel rounds it: no empty split
    use_cluster = (CLUSTER_REDUCE if cluster is None else cluster) and swap and 2 <= splits <= CLUSTER_MAX and not fused_reduce
    pieces = pieces and splits > 1 and not fused_reduce and not use_cluster
    if normed is not None and (not swap or bn > 64):
        raise KernelError("gemm_tc: a normed input needs the few-token order")
    ssq = None
    if residual is not None:
        if not use_cluster or gated or N % 4:
            raise KernelError("gemm_tc: the residual add needs 2..8 K ranges summed inside a cluster (see can_add_residual)")
        if residual.dtype != torch.float32 or residual.shape != (T, N) or residual.stride(1) != 1 or residual.stride(0) % 4:
            raise KernelError("gemm_tc: residual must be float32 [T, N] with unit inner stride")
        ssq = torch.empty((T, -(-N // 128)), dtype=torch.float32, device=dev)
    if gated:
        if not swap or splits != 1 or N % 128 or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc: the gated epilogue needs the few-token order, one split, N % 128 == 0, bfloat16")
        if out is None:
            out = torch.empty((T, N // 2), dtype=out_dtype, device=dev)
        elif out.shape != (T, N // 2) or out.dtype != out_dtype or out.stride(1) != 1:
            raise KernelError("gemm_tc: out must be [T, N / 2] bfloat16 for the gated epilogue")
    elif pieces or residual is not None:
        out = None
    elif out is None:
        out = torch.empty((T, N), dtype=out_dtype, device=dev)
    elif out.shape != (T, N) or out.dtype != out_dtype or out.stride(1) != 1:
        raise KernelError("gemm_tc: out must be [T, N] of the output type with unit inner stride")
    partial = torch.empty((splits, T, N), dtype=torch.float32, device=dev) if splits > 1 and not use_cluster else None
    st = status_word(dev)
    ldo = N if out is None else out.stride(0)
    name = (f"gemm_tc<{bn}>" + ("+gated" if gated else "") + ("+cluster" if use_cluster else "") + ("+pieces" if pieces else "")
            + ("" if swap else "+rows") + ("+normed" if normed is not None else "") + ("+residual" if residual is not None else ""))
    launches = 1 if (splits == 1 or fused_reduce or pieces or use_cluster) else 2
    counters = (st.data_ptr() + 4) if fused_reduce else None
    if normed is None and residual is None:
        _check(lib().tl_gemm_tc(_ptr(x), _ptr(w), _ptr(out), int(out_dtype == torch.float32), ldo, T, N, K, swap, bn, splits,
                                _ptr(partial), _ptr(st), counters, N_COUNTERS, int(gated), int(use_cluster), _stream()),
               name, launches=launches)
    else:
        n = normed
        _check(lib().tl_gemm_tc_normed(
            _ptr(x), _ptr(w), _ptr(out), int(out_dtype == torch.float32), ldo, T, N, K, swap, bn, splits,
            _ptr(partial), _ptr(st), counters, N_COUNTERS, int(gated), int(use_cluster),
            _ptr(residual), residual.stride(0) if residual is not None else 0, _ptr(ssq),
            _ptr(n.x) if n else None, _ptr(n.ssq) if n else None, n.ssq.shape[1] if n else 0, _ptr(n.weight) if n else None,
            int(n.weight.dtype == torch.float32) if n else 0, float(n.eps) if n else 0.0, _stream()), name, launches=launches)
    if residual is not None:
        return ssq
    return partial if pieces else out


_lib2 = None


def lib2():
    """The two-block (cta_group::2) persistent product for steps of many tokens (`csrc/gemm_tc2.cu`)."""
    global _lib2
    if _lib2 is None:
        l = load_library("tl_gemm_tc2", ["gemm_tc2.cu"])
        l.tl_gemm_tc2.argtypes = [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P]
        l.tl_gemm_tc2.restype = ctypes.c_int
        _lib2 = l
    return _lib2


def gemm_tc2(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, *, gated: bool = False,
             out: torch.Tensor | None = None, max_pairs: int = 0) -> torch.Tensor:
    """x [T, K] times w [N, K]^T on pairs of thread blocks (256 x 256 tiles, persistent, double-buffered
    accumulators).  `gated`: w holds gate and up rows interleaved in blocks of 64 (N % 128 == 0); the result is
    silu(gate) * up, [T, N / 2] bfloat16, formed in the epilogue."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc2: bfloat16 operands only")
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not x.is_contiguous() or not w.is_contiguous():
        raise KernelError("gemm_tc2: x [T, K] and w [N, K] must be contiguous with equal K")
    if K % 8:
        raise KernelError(f"gemm_tc2: K = {K} must be a multiple of 8 (TMA needs 16-byte rows)")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tc2: output is bfloat16 or float32")
    if gated and (N % 128 or out_dtype != torch.bfloat16):
        raise KernelError("gemm_tc2: the gated epilogue needs N % 128 == 0 and bfloat16 output")
    cols = N // 2 if gated else N
    if out is None:
        out = torch.empty((T, cols), dtype=out_dtype, device=x.device)
    elif out.shape != (T, cols) or out.dtype != out_dtype or out.stride(1) != 1:
        raise KernelError("gemm_tc2: out must be [T, N] (gated: [T, N / 2]) of the output type with unit inner stride")
    st = status_word(x.device)
    _check(lib2().tl_gemm_tc2(_ptr(x), _ptr(w), _ptr(out), int(out_dtype == torch.float32), out.stride(0), T, N, K,
                              int(gated), _ptr(st), int(max_pairs), _stream()), "gemm_tc2" + ("+gated" if gated else ""))
    return out


def can_gate(T: int, N: int, K: int) -> bool:
    """Whether the plan for these sizes allows the gated epilogue."""
    swap, _, splits = plan(T, N, K)
    return bool(swap) and splits == 1 and N % 128 == 0


def sum_pieces(pieces: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """[S, T, N] float32 pieces of a split-K product -> their sum in split order, [T, N]."""
    S, T, N = pieces.shape
    out = torch.empty((T, N), dtype=out_dtype, device=pieces.device)
    _check(lib().tl_splitk_reduce(_ptr(pieces), _ptr(out), int(out_dtype == torch.float32), S, T, N, N, _stream()),
           "splitk_reduce")
    return out

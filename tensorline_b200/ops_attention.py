"""Launchers of the tensor-core attention kernels (bfloat16), built per head size.

`attend_bf16` picks the kernel for a step: steps of single decoded tokens use the split-KV decode
kernel (with its combine pass when the keys are split), every other step uses the prefill kernel,
which also serves decoded tokens that ride along with prompt portions.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .csrc.build import load_library
from . import ops
from .ops import KernelError, _check, _ptr, _stream

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_libs: dict = {}

KEY_TILE = 64
DECODE_MAX_TABLE_ENTRIES = 1024     # block-table entries a decode block copies to shared memory (`tl_attn_decode_max_table`)
TC_PREFILL = os.environ.get("TENSORLINE_B200_TC", "1") != "0"   # 0: mma.sync attention only (A/B timing)


def attn_lib(head_dim: int):
    """The attention library compiled for this head size (built at first use)."""
    lib = _libs.get(head_dim)
    if lib is None:
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise KernelError(f"head_dim {head_dim}: the bfloat16 attention kernels take multiples of 16 "
                              "from 16 to 256")
        defines = {"HEAD_DIM": head_dim}
        if os.environ.get("TL_DEC_STAGES"):
            defines["TL_DEC_STAGES"] = int(os.environ["TL_DEC_STAGES"])
        lib = load_library(f"tl_attn_hd{head_dim}", ["attn_mma.cu"], defines)
        lib.tl_attn_prefill.argtypes = [_P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _I, _I, _P, _P]
        lib.tl_attn_prefill.restype = ctypes.c_int
        lib.tl_attn_decode.argtypes = [_P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, _I, _I, _P, _P]
        lib.tl_attn_decode.restype = ctypes.c_int
        lib.tl_attn_decode_tma.argtypes = [_P, _I, _P, _P, _P, ctypes.c_longlong, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I,
                                           _F, _I, _I, _P, _P, _P, _I, _I, _P, _P]
        lib.tl_attn_decode_tma.restype = ctypes.c_int
        lib.tl_attn_decode_tma_rope.argtypes = lib.tl_attn_decode_tma.argtypes[:-1] + [_P, _P, _I, _I, _P]
        lib.tl_attn_decode_tma_rope.restype = ctypes.c_int
        if lib.tl_attn_decode_max_table() != DECODE_MAX_TABLE_ENTRIES:
            raise KernelError(f"the attention library copies {lib.tl_attn_decode_max_table()} block-table entries a block, "
                              f"the split planner assumes {DECODE_MAX_TABLE_ENTRIES}")
        _libs[head_dim] = lib
    return lib


def decode_blocks_per_sm(head_dim: int) -> int:
    """Decode blocks that fit one SM: three stages of 64 keys and values, rows padded by 8 elements."""
    stages = int(os.environ.get("TL_DEC_STAGES", 3))
    smem = 16 * (head_dim + 8) * 2 + max(2 * stages * KEY_TILE * (head_dim + 8) * 2, (4 * 16 * head_dim + 128) * 4) + 2048
    return max(1, min(3, (227 * 1024) // (smem + 1024)))


_tc_libs: dict = {}
TC_QUERY_TILE = 128


def attn_tc_lib(head_dim: int):
    """The tcgen05 prefill attention compiled for this head size (64, 128, 192 or 256)."""
    lib = _tc_libs.get(head_dim)
    if lib is None:
        if head_dim % 64 or not 64 <= head_dim <= 256:
            raise KernelError(f"head_dim {head_dim}: the tcgen05 attention kernel takes 64, 128, 192 or 256")
        lib = load_library(f"tl_attn_tc_hd{head_dim}", ["attn_tc.cu"], {"HEAD_DIM": head_dim})
        lib.tl_attn_tc_prefill.argtypes = [_P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P, _I, _I, _P, _P]
        lib.tl_attn_tc_prefill.restype = ctypes.c_int
        lib.tl_attn_tc2_prefill.argtypes = [_P, _I, _P, _P, _P, ctypes.c_longlong, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _F,
                                            _I, _P, _P, _I, _P, _P]
        lib.tl_attn_tc2_prefill.restype = ctypes.c_int
        lib.tl_attn_tc3_prefill.argtypes = lib.tl_attn_tc2_prefill.argtypes
        lib.tl_attn_tc3_prefill.restype = ctypes.c_int
        lib.tl_attn_tc2p_prefill.argtypes = lib.tl_attn_tc2_prefill.argtypes
        lib.tl_attn_tc2p_prefill.restype = ctypes.c_int
        lib.tl_attn_tc2_prefill_split.argtypes = lib.tl_attn_tc2_prefill.argtypes[:-1] + [_I, _I, _I, _P, _P, _P, _I, _P]
        lib.tl_attn_tc2_prefill_split.restype = ctypes.c_int
        _tc_libs[head_dim] = lib
    return lib


def tc_min_page(head_dim: int) -> int:
    """One warp hands the page numbers of a 64-key tile around by shuffle: at most 32 pages per tile."""
    return 2


def prefill_tc(q, q_stride, out, k_pages, v_pages, table, page_size, q_start, start_pos, slots, h_q_start,
               nq, nkv, d, window, scale, order=None) -> None:
    """Prompt-portion attention on tcgen05: 128 query rows per block, S and O in tensor memory."""
    from .ops_gemm import status_word
    if page_size < tc_min_page(d) or page_size > KEY_TILE or page_size & (page_size - 1):
        raise KernelError(f"page size {page_size}: the tcgen05 attention kernel for head size {d} takes powers of two "
                          f"from {tc_min_page(d)} to {KEY_TILE}")
    g = nq // nkv
    B = len(h_q_start) - 1
    tiles = sum(-(-(h_q_start[i + 1] - h_q_start[i]) * g // TC_QUERY_TILE) for i in range(B))
    if order is not None:
        tiles = order.numel()                           # the array may leave requests out
    _check(attn_tc_lib(d).tl_attn_tc_prefill(_ptr(q), q_stride, _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(table),
                                             table.shape[1], page_size, _ptr(q_start), _ptr(start_pos), _ptr(slots), B,
                                             nq, nkv, int(window or 0), float(scale), tiles,
                                             _ptr(status_word(q.device)), _ptr(order) if order is not None else None,
                                             table.shape[0], k_pages.shape[0], ops.fault_words(q.device),
                                             _stream()), "attn_tc_prefill")


def tile_order(h_q_start, h_start_pos, group: int, rows_per_tile: int, device, skip=()):
    """The order in which a prompt-portion kernel's blocks take the query tiles of a step with several requests:
    int32 (request << 16 | tile), the tile that reads the most keys first, so that the long tiles of every request
    start in the first round of blocks and the short ones fill the end.  Requests in `skip` get no tile (another
    kernel serves them).  None for one request and nothing to skip (the kernel's own order, last tile first, is
    the same) or when the numbers do not fit 16 bits."""
    B = len(h_q_start) - 1
    if (B <= 1 and not skip) or B >= 1 << 15:
        return None
    tiles = []
    for b in range(B):
        if b in skip:
            continue
        rows = (h_q_start[b + 1] - h_q_start[b]) * group
        n = -(-rows // rows_per_tile)
        if n >= 1 << 16:
            return None
        for t in range(n):
            last_token = min(rows, (t + 1) * rows_per_tile) - 1
            tiles.append((-(h_start_pos[b] + last_token // group + 1), b, t))
    tiles.sort()
    return torch.tensor([(b << 16) | t for _, b, t in tiles], dtype=torch.int32).to(device, non_blocking=True)


TILE_ORDER = os.environ.get("TENSORLINE_B200_TILE_ORDER", "1") != "0"   # 0: request after request (A/B timing)
TC_PAIR = os.environ.get("TENSORLINE_B200_TC_PAIR", "1") != "0"   # 0: one query tile per block only (A/B timing)
KEY_SPLIT = os.environ.get("TENSORLINE_B200_KEY_SPLIT", "1") != "0"   # 0: a query tile's keys never dealt out to several blocks


# Where the pair kernel keeps P.  "64" (default): the softmax writes P back into the S slot it has read (tensor memory)
# and O += P V takes it from there; key tiles of 64, two S slots a query tile.  Bit for bit the results of "0" (P through
# shared memory) and 1 to 4 % faster at 2,048 and 4,096 tokens (46.5 -> 45.5, 142 -> 139 us at 7B head counts, 69.5 ->
# 66.7 at 14B), equal at 8,192: the step is bound by the softmax warps' instructions, not by shared memory.  "1": key
# tiles of 128 and one S slot a query tile; correct (same tests) but slower (8,192 tokens: 916 against 512 us): a tile's
# products and softmax alternate and the softmax of 128 keys a row is the whole step.  Kept for further work.
TC_P_IN_TMEM = {"0": False, "1": True}.get(os.environ.get("TENSORLINE_B200_TC_P_TMEM", "64"), "64")


def prefill_tc_pair(q, q_stride, out, k_pages, v_pages, table, page_size, q_start, start_pos, slots, h_q_start,
                    nq, nkv, d, window, scale, order=None, p_in_tmem=None, ksplit: int = 1, merge_rows=None) -> bool:
    """Prompt-portion attention on tcgen05 with two query tiles (256 rows) per block and K, V by TMA.
    `p_in_tmem` (None: as the switch says): "64": P kept in tensor memory, key tiles of 64; False: P through shared
    memory; True: key tiles of 128 and P in tensor memory.  Head sizes 64 and 128, pages of 8 to 64 tokens; returns
    False (nothing launched) for other sizes.
    `ksplit` (2..8, not with the 128-key kernel): every block's key tiles are dealt out to that many blocks and a second
    kernel merges their parts; `merge_rows`: int32 device tensor of the tokens this launch serves (None: all rows of
    `out`).  For portions on long contexts whose query tiles alone leave most of the GPU idle."""
    from .ops_gemm import status_word
    p_in_tmem = TC_P_IN_TMEM if p_in_tmem is None else p_in_tmem
    if d > 128 or page_size < 8 or page_size > KEY_TILE or page_size & (page_size - 1):
        return False
    g = nq // nkv
    B = len(h_q_start) - 1
    tiles = sum(-(-(h_q_start[i + 1] - h_q_start[i]) * g // (2 * TC_QUERY_TILE)) for i in range(B))
    if order is not None:
        tiles = order.numel()
    lib = attn_tc_lib(d)
    if ksplit > 1 and p_in_tmem is not True:
        T = out.shape[0]
        if merge_rows is None:
            merge_rows = torch.arange(T, dtype=torch.int32, device=q.device)
        part_o = torch.empty((ksplit, T, nq, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((ksplit, T, nq, 2), dtype=torch.float32, device=q.device)
        rc = lib.tl_attn_tc2_prefill_split(
            _ptr(q), q_stride, _ptr(out), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(table), table.shape[1], page_size,
            _ptr(q_start), _ptr(start_pos), _ptr(slots), B, nq, nkv, int(window or 0), float(scale), tiles,
            _ptr(status_word(q.device)), _ptr(order) if order is not None else None, table.shape[0], ops.fault_words(q.device),
            int(p_in_tmem == "64"), ksplit, T, _ptr(part_o), _ptr(part_ml), _ptr(merge_rows), merge_rows.numel(), _stream())
        if rc == 2:
            return False
        _check(rc, "attn_tc2_prefill+split", launches=2)
        return True
    entry = lib.tl_attn_tc2p_prefill if p_in_tmem == "64" else lib.tl_attn_tc3_prefill if p_in_tmem is True else lib.tl_attn_tc2_prefill
    rc = entry(_ptr(q), q_stride, _ptr(out), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0],
                                            _ptr(table), table.shape[1], page_size, _ptr(q_start), _ptr(start_pos),
                                            _ptr(slots), B, nq, nkv, int(window or 0), float(scale), tiles,
                                            _ptr(status_word(q.device)), _ptr(order) if order is not None else None,
                                            table.shape[0], ops.fault_words(q.device), _stream())
    if rc == 2:
        return False
    _check(rc, "attn_tc3_prefill" if p_in_tmem is True else "attn_tc2_prefill")     # "64" is the same kernel, another place for P
    return True


def plan_splits(batch: int, nkv: int, group: int, span: int, head_dim: int = 128, max_splits: int = 128,
                page_size: int = 16, sms: int | None = None) -> tuple:
    """(chunk, splits) for a decode step; `span` is the largest number of keys a request can read.
    A block streams its range of keys tile by tile (64 keys), and a tile costs it about a microsecond
    whatever else runs, so a request's keys are cut into ranges until the blocks fill the GPU's resident
    slots once (a second, partly filled round would double the time) - but not finer than four tiles a
    range (two when that leaves 64 blocks or fewer), below which the merge of the partials costs more
    than the shorter ranges save.  Measured at 7B sizes, context 4,090: batch 1 to 3 -> 16 ranges (one cluster of sixteen blocks a (request, KV head)), 4 to 8 -> 8,
    16 -> 4, 32 -> 2, 64 -> 1.
    A block copies its range's block-table entries to shared memory, DECODE_MAX_TABLE_ENTRIES at most: a range is
    never longer than that many pages, whatever the rules above say (long contexts on small pages get more ranges)."""
    NUM_SMS = sms or ops.num_sms()
    m_tiles = -(-group // 16)
    tiles = max(1, -(-span // KEY_TILE))
    base = max(1, batch * nkv * m_tiles)
    resident = NUM_SMS * decode_blocks_per_sm(head_dim)
    fill = max(1, resident // base)
    splits = min(fill, max(1, tiles // 4), max_splits)
    if base * splits <= 64:
        splits = min(fill, max(1, tiles // 2), max_splits)
    if splits > 8 and base <= CLUSTER16_MAX and m_tiles == 1:
        # few requests: sixteen ranges in a cluster of sixteen blocks (no parts in memory, no combine kernel, which alone
        # cost 5 us a layer at batch 1)
        splits = min(splits, 16)
    elif 8 < splits <= 16:
        # eight ranges merge inside a cluster; measured at batch 8, 8 k to 32 k keys: 27 / 46 / 86 against 30 / 49 / 88 us
        # with nine; at batch 2 and 4, context 4,090, against sixteen ranges and the combine kernel: 2.768 / 2.793 against
        # 2.782 / 2.861 ms a step
        splits = 8
    chunk = -(-tiles // splits) * KEY_TILE
    most = max(KEY_TILE, DECODE_MAX_TABLE_ENTRIES * page_size // KEY_TILE * KEY_TILE)
    chunk = min(chunk, most)
    splits = -(-tiles * KEY_TILE // chunk)
    return chunk, splits


def prefill(q, q_stride, out, k_pages, v_pages, table, page_size, q_start, start_pos, slots, h_q_start,
            nq, nkv, d, window, scale, order=None) -> None:
    g = nq // nkv
    B = len(h_q_start) - 1
    tiles = sum(-(-(h_q_start[i + 1] - h_q_start[i]) * g // KEY_TILE) for i in range(B))
    if order is not None:
        tiles = order.numel()
    if KEY_TILE % page_size:
        raise KernelError(f"page size {page_size} must divide {KEY_TILE}")
    _check(attn_lib(d).tl_attn_prefill(_ptr(q), q_stride, _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(table),
                                       table.shape[1], page_size, _ptr(q_start), _ptr(start_pos), _ptr(slots), B,
                                       nq, nkv, int(window or 0), float(scale), tiles,
                                       _ptr(order) if order is not None else None, table.shape[0], k_pages.shape[0],
                                       ops.fault_words(q.device), _stream()), "attn_prefill")


CLUSTER16_MAX = int(os.environ.get("TENSORLINE_B200_CLUSTER16_MAX", "12"))   # (request, KV head) pairs up to which 16 ranges merge in a cluster; 0: never
TMA_DECODE = os.environ.get("TENSORLINE_B200_TMA_DECODE", "1") != "0"   # 0: cp.async loads only (A/B timing)
TMA_DECODE_MIN_BATCH = int(os.environ.get("TENSORLINE_B200_TMA_DECODE_MIN_BATCH", "1"))   # fewer requests: cp.async loads
CLUSTER_MERGE = os.environ.get("TENSORLINE_B200_CLUSTER_MERGE", "1") != "0"   # 0: partials + combine kernel (A/B timing)


FOLD_ROPE = os.environ.get("TENSORLINE_B200_FOLD_ROPE", "1") != "0"   # 0: the rotary step always a kernel of its own (A/B timing)


def decode_takes_rope(B: int, d: int, page_size: int) -> bool:
    """Whether a decode step of these sizes goes to the kernel that can do bias, rotation and the page write of the
    step's own tokens itself (the TMA decode kernel, as `decode` picks it)."""
    return FOLD_ROPE and TMA_DECODE and B >= TMA_DECODE_MIN_BATCH and d % 64 == 0 and 8 <= page_size <= 64 and page_size & (page_size - 1) == 0


def decode(q, q_stride, out, k_pages, v_pages, table, page_size, q_start, start_pos, slots, B,
           nq, nkv, d, window, scale, chunk, splits, part_o=None, part_ml=None, tma: bool | None = None,
           cluster: bool | None = None, rope: dict | None = None) -> None:
    """Split-KV decode attention.  `tma`: load K and V by TMA (head sizes that are multiples of 64, pages of
    8..64 tokens); None = wherever that applies.  `cluster` (TMA path, 2..8 key ranges, groups of at most 16
    heads): the ranges of a request merge inside a thread-block cluster, no partials, no second kernel;
    None = wherever that applies.
    `rope` (TMA path only; see `decode_takes_rope`): `q` is the step's q|k|v as the projection left it and the kernel
    does bias, rotation and the page write itself: {"inv_freq", "bias" (or None), "write_kv", "unfold"}; `unfold()`
    runs the rotary kernel instead, for the case that the library turns the launch down."""
    if KEY_TILE % page_size:
        raise KernelError(f"page size {page_size} must divide {KEY_TILE}")
    use_tma = (TMA_DECODE and B >= TMA_DECODE_MIN_BATCH if tma is None else tma) and d % 64 == 0 and 8 <= page_size <= 64
    if rope is not None and not use_tma:
        raise KernelError("attn_decode: the rotary step folds into the TMA kernel only")
    # up to 8 ranges in a cluster of the portable size; 9 to 16 (this GPU's limit) while the clusters are few enough to be
    # placed at once (14 of them fit)
    can_cluster = use_tma and nq // nkv <= 16 and (2 <= splits <= 8 or (9 <= splits <= 16 and B * nkv <= CLUSTER16_MAX))
    use_cluster = can_cluster and (CLUSTER_MERGE if cluster is None else cluster)
    if splits > 1 and not use_cluster:
        if part_o is None or part_o.numel() < B * nq * splits * d or part_o.dtype != torch.float32:
            raise KernelError("attn_decode: part_o must be float32 [B, nq, splits, d]")
        if part_ml is None or part_ml.numel() < B * nq * splits * 2 or part_ml.dtype != torch.float32:
            raise KernelError("attn_decode: part_ml must be float32 [B, nq, splits, 2]")
    # measured at 7B sizes: TMA loads win at batch 64 (5.8 against 5.4 TB/s); with fewer requests the loads themselves
    # make no difference, but the TMA kernel can take the rotary step in and start its loads before the kernel in
    # front has finished (batch 1: 2.85 -> 2.80 ms a step)
    if use_tma:
        from .ops_gemm import status_word
        args = (_ptr(q), q_stride, _ptr(out), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0],
                _ptr(table), table.shape[1], page_size, _ptr(q_start), _ptr(start_pos),
                _ptr(slots), B, nq, nkv, int(window or 0), float(scale), chunk, splits,
                _ptr(part_o) if splits > 1 and not use_cluster else None,
                _ptr(part_ml) if splits > 1 and not use_cluster else None,
                _ptr(status_word(q.device)), int(use_cluster), table.shape[0], ops.fault_words(q.device))
        if rope is not None:
            bias = rope["bias"]
            rc = attn_lib(d).tl_attn_decode_tma_rope(*args, _ptr(rope["inv_freq"]), _ptr(bias),
                                                     int(bias is not None and bias.dtype == torch.float32),
                                                     int(rope["write_kv"]), _stream())
        else:
            rc = attn_lib(d).tl_attn_decode_tma(*args, _stream())
        if rc != 2:                                    # 2: this build or these sizes do not take the TMA path
            _check(rc, "attn_decode_tma" + ("+rope" if rope is not None else "") + ("+cluster" if use_cluster else "+combine" if splits > 1 else ""),
                   launches=2 if splits > 1 and not use_cluster else 1)
            return
        if rope is not None:                           # turned down: the rotary step as a kernel of its own after all
            rope["unfold"]()
    _check(attn_lib(d).tl_attn_decode(_ptr(q), q_stride, _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(table),
                                      table.shape[1], page_size, _ptr(q_start), _ptr(start_pos), _ptr(slots), B,
                                      nq, nkv, int(window or 0), float(scale), chunk, splits,
                                      _ptr(part_o) if splits > 1 else None, _ptr(part_ml) if splits > 1 else None,
                                      table.shape[0], k_pages.shape[0], ops.fault_words(q.device),
                                      _stream()), "attn_decode" + ("+combine" if splits > 1 else ""), launches=2 if splits > 1 else 1)


def attend_bf16(qkv, o, ctx, k_pages, v_pages, table, nq, nkv, d, window, scale, rope: dict | None = None) -> None:
    """`rope`: only for decode-only steps that `decode_takes_rope` accepted (see `decode`)."""
    if qkv.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        raise KernelError("attend_bf16: bfloat16 tensors only")
    q_stride = qkv.shape[1]
    if rope is not None and not ctx.decode_only:
        raise KernelError("attend_bf16: the rotary step folds into decode-only steps")
    if ctx.decode_only:
        span = ctx.graph_max_ctx or ctx.max_ctx
        if window:
            span = min(span, window + KEY_TILE - 1)
        chunk, splits = plan_splits(ctx.B, nkv, nq // nkv, span, d, page_size=ctx.page_size)
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((ctx.B, nq, splits, d), dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty((ctx.B, nq, splits, 2), dtype=torch.float32, device=qkv.device)
        decode(qkv, q_stride, o, k_pages, v_pages, table, ctx.page_size, ctx.q_start, ctx.start_pos, ctx.slots,
               ctx.B, nq, nkv, d, window, scale, chunk, splits, part_o, part_ml, rope=rope)
    else:
        g = nq // nkv
        singles = _single_token_requests(ctx, qkv.device, g, nkv)
        skip = singles["set"] if singles else frozenset()
        if singles:
            # the single decoded tokens of a mixed step: the decode kernel cuts their keys into ranges, where a
            # query tile of the portion kernels would walk one request's whole context with 1 row in 18 used
            span = min(singles["span"], window + KEY_TILE - 1) if window else singles["span"]
            n = len(skip)
            chunk, splits = plan_splits(n, nkv, g, span, d, page_size=ctx.page_size)
            part_o = part_ml = None
            if splits > 1:
                part_o = torch.empty((n, nq, splits, d), dtype=torch.float32, device=qkv.device)
                part_ml = torch.empty((n, nq, splits, 2), dtype=torch.float32, device=qkv.device)
            # The two kernels read the same inputs and write different rows, and neither fills the GPU alone (the
            # portion's blocks are few and bound by arithmetic, the decode kernel is bound by memory): the decode
            # kernel goes to a second stream and the step's stream joins it after the portion kernel.
            joined = None
            if SINGLES_STREAM and qkv.is_cuda:
                main, side = torch.cuda.current_stream(qkv.device), _side_stream(qkv.device)
                ready = torch.cuda.Event()
                ready.record(main)                         # the step's q, k, v and pages are complete
                with torch.cuda.stream(side):
                    side.wait_event(ready)
                    decode(qkv, q_stride, o, k_pages, v_pages, table, ctx.page_size, singles["rows"], singles["start_pos"],
                           singles["slots"], n, nq, nkv, d, window, scale, chunk, splits, part_o, part_ml)
                    joined = torch.cuda.Event()
                    joined.record(side)
            else:
                decode(qkv, q_stride, o, k_pages, v_pages, table, ctx.page_size, singles["rows"], singles["start_pos"],
                       singles["slots"], n, nq, nkv, d, window, scale, chunk, splits, part_o, part_ml)
        rest = [i for i in range(ctx.B) if i not in skip]
        rest_rows = sum(ctx.h_q_start[i + 1] - ctx.h_q_start[i] for i in rest) * g
        # Steps whose requests bring enough query rows to fill 128-row tiles run on tcgen05, and so do steps with a
        # portion of a thousand rows or more whatever else is beside it (a 464-token portion beside 48 single tokens,
        # 14B head counts: 129 against 169 us); steps of mostly single tokens beside a short portion keep the 64-row
        # mma.sync tiles.
        use_tc = TC_PREFILL and d % 64 == 0 and d <= 256 and ctx.page_size >= tc_min_page(d) and \
            (rest_rows >= 96 * len(rest) or rest_rows >= 8 * TC_QUERY_TILE)
        args = (qkv, q_stride, o, k_pages, v_pages, table, ctx.page_size, ctx.q_start, ctx.start_pos, ctx.slots,
                ctx.h_q_start, nq, nkv, d, window, scale)
        # Two query tiles a block pay as soon as the one-tile kernel's blocks (one an SM) would need a second round:
        # measured at 7B head counts 2,048 new tokens 45 against 71 us, 1,024 on 1,024 cached (224 one-tile blocks) 46
        # against 58 us, but 512 on 3,584 cached (112 blocks) 76 against 70 us; at 14B head counts 512 on 1,024 cached
        # (160 blocks) 36 against 47 us, 512 on 3,584 cached 78 against 121 us, 256 on 1,024 cached (80 blocks) 31
        # against 29 us.
        one_tile_blocks = sum(-(-(ctx.h_q_start[i + 1] - ctx.h_q_start[i]) * g // TC_QUERY_TILE) for i in rest) * nkv

        def order(rows_per_tile):
            if not TILE_ORDER and not skip:
                return None
            key = ("tile_order", g, rows_per_tile)
            if key not in ctx.scratch:
                ctx.scratch[key] = tile_order(ctx.h_q_start, ctx.h_start_pos, g, rows_per_tile, qkv.device, skip)
            return ctx.scratch[key]
        # A portion on a long context whose pairs of query tiles fill less than half the GPU: every block's key tiles
        # are dealt out to several blocks and their parts merged by a second kernel (7B head counts, 512 tokens on
        # 3,584 cached: 54 against 71 us for the one-tile kernel and 77 for the pair kernel alone; 256 tokens: 35
        # against 66; 128 tokens on 8,000 cached: 42 against 127), as long as a run keeps twelve key tiles or more.
        ksplit = 1
        if use_tc and TC_PAIR and KEY_SPLIT and d <= 128 and not window:
            pair_blocks = sum(-(-(ctx.h_q_start[i + 1] - ctx.h_q_start[i]) * g // (2 * TC_QUERY_TILE)) for i in rest) * nkv
            key_tiles = max(-(-(ctx.h_start_pos[i] + ctx.h_q_start[i + 1] - ctx.h_q_start[i]) // KEY_TILE) for i in rest) if rest else 0
            ksplit = min(8, ops.num_sms() // max(1, pair_blocks), key_tiles // 12)
        if ksplit >= 2:
            rows_key = ("merge_rows", len(skip))
            if rows_key not in ctx.scratch:
                rows = [t for i in rest for t in range(ctx.h_q_start[i], ctx.h_q_start[i + 1])]
                ctx.scratch[rows_key] = torch.tensor(rows, dtype=torch.int32).to(qkv.device, non_blocking=True)
            if not prefill_tc_pair(*args, order(2 * TC_QUERY_TILE), ksplit=ksplit, merge_rows=ctx.scratch[rows_key]):
                ksplit = 1
        if ksplit >= 2:
            pass
        elif use_tc and TC_PAIR and one_tile_blocks > ops.num_sms() and prefill_tc_pair(*args, order(2 * TC_QUERY_TILE)):
            pass
        elif use_tc:
            prefill_tc(*args, order(TC_QUERY_TILE))
        else:
            prefill(*args, order(KEY_TILE))
        if singles and joined is not None:
            torch.cuda.current_stream(qkv.device).wait_event(joined)


SINGLES_STREAM = os.environ.get("TENSORLINE_B200_SINGLES_STREAM", "1") != "0"   # 0: both kernels on the step's stream (A/B timing)
_side_streams: dict = {}


def _side_stream(device):
    """The second stream of `device` for the single tokens of mixed steps (one for the life of the process)."""
    key = torch.device(device).index
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


SINGLES_MIN_KEYS = int(os.environ.get("TENSORLINE_B200_SINGLES_MIN_KEYS", 768))
SINGLES_RATIO = float(os.environ.get("TENSORLINE_B200_SINGLES_RATIO", 1.5))
SINGLES_FILL = float(os.environ.get("TENSORLINE_B200_SINGLES_FILL", 1.6))


def _single_token_requests(ctx, device, group: int, nkv: int = 1, sms: int | None = None):
    """The requests of a mixed step that bring one token, if they are worth a launch of the decode kernel: the longest
    of them reads SINGLES_MIN_KEYS keys or more and either SINGLES_RATIO times as many as any other request of the step
    (a query tile walks its keys alone, so the longest one sets the pace of the portion kernel; measured at 7B sizes,
    a layer: 7 x 4,000 cached beside 2,041 new tokens 66 against 83 us, 3 x 8,000 beside 509 33 against 156 us, 31
    x 1,000 beside 481 30 against 35 us, but 3,000 / 2,000 / 500 beside 2,045 66 against 62 us and 7 x 4,000 beside
    2,041 on 2,048 cached 122 against 115 us), or there are so many of them that their (request, KV head) pairs fill
    the GPU SINGLES_FILL times over: the decode kernel streams keys faster than a query tile with one token in it
    (a 464-token portion beside 48 single tokens at 1,500 keys, 8 KV heads: 105 against 129 us; beside 16: 80 against
    72; 4 KV heads, 48 single tokens: 82 against 72).  {"set", "rows", "start_pos", "slots", "span"} with device tensors,
    or None.  Computed once a step."""
    key = ("single_token_requests", group, nkv)
    if key not in ctx.scratch:
        B = ctx.B
        ones = [b for b in range(B) if ctx.h_q_start[b + 1] - ctx.h_q_start[b] == 1]
        found = None
        span = max((ctx.h_start_pos[b] + 1 for b in ones), default=0)
        rest_span = max((ctx.h_start_pos[b] + ctx.h_q_start[b + 1] - ctx.h_q_start[b] for b in range(B)
                         if ctx.h_q_start[b + 1] - ctx.h_q_start[b] != 1), default=0)
        many = len(ones) * nkv >= SINGLES_FILL * (sms or ops.num_sms()) if len(ones) * nkv >= 64 else False
        if ones and len(ones) < B and B < 1 << 15 and span >= SINGLES_MIN_KEYS and (span >= SINGLES_RATIO * rest_span or many) and \
                all((ctx.h_q_start[b + 1] - ctx.h_q_start[b]) * group < KEY_TILE << 16 for b in range(B)):
            n = len(ones)
            # longest context first: the decode kernel's blocks start in this order, one (request, KV head) each when
            # the GPU is full, and a long one that started last would run on alone
            ones.sort(key=lambda b: -ctx.h_start_pos[b])
            packed = torch.tensor([ctx.h_q_start[b] for b in ones] + [ctx.h_start_pos[b] for b in ones] +
                                  [ctx.h_slots[b] for b in ones], dtype=torch.int32).to(device, non_blocking=True)
            found = {"set": frozenset(ones), "rows": packed[:n], "start_pos": packed[n:2 * n], "slots": packed[2 * n:],
                     "span": span}
        ctx.scratch[key] = found
    return ctx.scratch[key]

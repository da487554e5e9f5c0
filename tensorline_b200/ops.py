"""Python launchers of the hand-written CUDA kernels.

Each function checks shapes, types and contiguity, then calls the C entry point of the compiled
library with raw device pointers on torch's current stream.  There is no CPU path and no library
stand-in: a CPU tensor or a missing library raises.
"""
from __future__ import annotations

import collections
import ctypes

import torch

from .csrc.build import CHECK_BUILD, load_library

CORE_SOURCES = ["elementwise.cu", "rope_kv.cu", "attn_tokenwise.cu", "gemm_f32.cu", "sampling.cu"]

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

_SIGNATURES = {
    "tl_embed": [_P, _P, _I, _P, _I, _I, _P],
    "tl_add_rmsnorm": [_P, _P, _P, _I, _P, _I, _P, _I, _I, _F, _I, _P, _I, ctypes.c_longlong, _P],
    "tl_silu_mul": [_P, _P, _I, _I, _I, _I, _P],
    "tl_rope_kv_write": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _P, _P, _I, _I, _P, _I, ctypes.c_longlong,
                         _I, _P, _P, _F, _I, _I, _P, _P],
    "tl_attn_tokenwise": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "tl_gemm_f32": [_P, _I, _P, _I, _I, _P, _P, _I, _I, _I, _I, _P],
    "tl_argmax": [_P, _I, _I, _I, _P, _P, _P],
    "tl_sample": [_P, _I, _I, _I, _P, _P, _P, _P, _P],
}


class KernelError(RuntimeError):
    pass


_core = None


def core():
    global _core
    if _core is None:
        lib = load_library("tl_core", CORE_SOURCES)
        for name, sig in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = sig
            fn.restype = ctypes.c_int
        _core = lib
    return _core


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dt}")


def _ptr(t: torch.Tensor | None):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernel called with a CPU tensor: this engine has no CPU path")
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


_launches = 0
kernel_counts: collections.Counter = collections.Counter()      # calls per kernel variant, by the name its launcher gives


def launch_count() -> int:
    """Kernels of this package launched so far in this process (a replayed CUDA graph counts the
    launches it holds)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str, launches: int = 1) -> None:
    global _launches
    if status != 0:
        raise KernelError(f"{what}: CUDA error {status} at launch")
    _launches += launches
    kernel_counts[what] += 1
    if _profile is not None:
        mark(what)


# ---------------------------------------------------------------------------------------------
# The device status word.  Kernels that wait on barriers (the tcgen05 products and attention, the TMA
# decode attention) bound every wait; a block whose wait runs out records a code here, stops and leaves
# output that is not valid.  The engine reads the word where the host waits for a step anyway (it
# travels with the sampled tokens) and fails the step's requests.

N_COUNTERS = 8192
_status: dict = {}
STATUS_ROLES = {1: "tcgen05 product: the copy thread waited for a free stage", 2: "tcgen05 product: the MMA thread waited for a stage's copies",
                3: "tcgen05 product: the epilogue waited for the accumulator",
                31: "two-block product: a copy thread waited for a free stage", 32: "two-block product: the MMA thread waited for a free accumulator",
                33: "two-block product: the MMA thread waited for a stage's copies", 34: "two-block product: the epilogue waited for the accumulator",
                20: "decode attention: a wait for a stage of keys and values"}


def device_status(device) -> torch.Tensor:
    """int32 [1 + N_COUNTERS + 4] on `device`: [0] is the status word (0 = no wait ran out), then the per-tile
    arrival counters of split products (zero between calls), then the four ints in which the checking build of the
    kernels records an index out of its bounds (code, kernel, value, limit)."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    t = _status.get(device)
    if t is None:
        with torch.inference_mode(False):                # an ordinary tensor: it is cleared in place from anywhere
            t = torch.zeros(1 + N_COUNTERS + 4, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def raise_device_status(device, code: int) -> None:
    """Clear the word and raise: a wait ran out inside a kernel."""
    device_status(device)[:1].zero_()
    what = STATUS_ROLES.get(int(code), "an attention kernel's pipeline wait" if int(code) >= 10 else "a pipeline wait")
    raise KernelError(f"a kernel on {device} gave up on a wait that did not complete in time (code {int(code)}: {what}); "
                      "the step's output is not valid")


KERNEL_NAMES = {1: "rotary + page write", 2: "exact-order attention", 3: "mma.sync prompt attention", 4: "decode attention",
                5: "TMA decode attention", 6: "tcgen05 prompt attention", 7: "two-tile tcgen05 prompt attention"}


def fault_words(device):
    """Device address of the four ints of the checking build, or None when the kernels are the ordinary build."""
    if not CHECK_BUILD:
        return None
    return device_status(device).data_ptr() + 4 * (1 + N_COUNTERS)


def check_device_status(device=None) -> None:
    """Raise if any kernel launched so far gave up on a wait or, in the checking build, met an index out of
    its bounds (synchronises; reads a few words per device that has them)."""
    for dev, t in list(_status.items()):
        if CHECK_BUILD:
            code, kernel, value, limit = t[1 + N_COUNTERS:].tolist()
            if code:
                t[1 + N_COUNTERS:].zero_()
                raise KernelError(f"bounds check on {dev}: the {KERNEL_NAMES.get(kernel, kernel)} kernel met index {value}, "
                                  f"which is outside [0, {limit}); the access went to the sink instead")
        code = int(t[0].item())
        if code:
            raise_device_status(dev, code)


def num_sms(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    dev = None if device is None else torch.device(device).index
    if dev is None:
        dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return n


_sm_counts: dict = {}


# ---------------------------------------------------------------------------------------------
# Profile: an event after every launch; the time between two events goes to the later one's name.

_profile = None


def start_profile() -> None:
    global _profile
    torch.cuda.synchronize()
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    _profile = [("start", first)]


def mark(name: str) -> None:
    """Inside a profile: everything launched since the last mark belongs to `name` (the launchers of this package
    call it themselves; callers of library kernels call it after them)."""
    if _profile is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        _profile.append((name, ev))


def stop_profile() -> dict:
    """name -> (calls, milliseconds) since `start_profile`."""
    global _profile
    marks, _profile = _profile, None
    torch.cuda.synchronize()
    out: dict = {}
    for (_, before), (name, ev) in zip(marks, marks[1:]):
        name = name.split("<")[0].split("+")[0] if name.startswith(("gemm_tc", "attn_")) else name
        calls, ms = out.get(name, (0, 0.0))
        out[name] = (calls + 1, ms + before.elapsed_time(ev))
    return out


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _ints(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")
    _contig(t, name)


# ---------------------------------------------------------------------------------------------

def embed(x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """x[t, :] = table[ids[t], :], x float32 [T, H]."""
    T, H = x.shape
    if x.dtype != torch.float32 or table.shape[1] != H or ids.numel() != T:
        raise KernelError("embed: x must be float32 [T, H] matching the table and ids")
    _contig(x, "x"); _contig(table, "table"); _ints(ids, "ids")
    _check(core().tl_embed(_ptr(x), _ptr(table), dtype_code(table.dtype), _ptr(ids), T, H, _stream()), "embed")


def add_rmsnorm(x: torch.Tensor, r: torch.Tensor | None, w: torch.Tensor, out: torch.Tensor, eps: float,
                rows: torch.Tensor | None = None, write_x: bool = True, pieces: torch.Tensor | None = None) -> None:
    """x += r (if r), out = cast(x * rstd) * w.  x float32 [*, H]; r, out of the activation
    type; `rows` picks the rows (x is then left alone).  `pieces` [S, rows of x, H] float32 instead
    of r: the addend as a split-K product left it; summed in split order and rounded to the
    activation type inside the kernel (needs H % 4 == 0 and H <= 32768)."""
    H = x.shape[-1]
    R = out.shape[0]
    if x.dtype != torch.float32 or out.shape[-1] != H or w.numel() != H:
        raise KernelError("add_rmsnorm: x must be float32 and out, w must match its width")
    if r is not None and (r.dtype != out.dtype or r.shape != x.shape):
        raise KernelError("add_rmsnorm: r must have x's shape and out's type")
    _contig(x, "x"); _contig(out, "out"); _contig(w, "w")
    if r is not None:
        _contig(r, "r")
    splits = plane = 0
    if pieces is not None:
        if r is not None or pieces.dtype != torch.float32 or pieces.dim() != 3 or pieces.shape[1:] != x.shape:
            raise KernelError("add_rmsnorm: pieces must be float32 [S, rows of x, H] and stand instead of r")
        if H % 4 or H > 32768:
            raise KernelError("add_rmsnorm: pieces need a width that is a multiple of 4 and at most 32768")
        _contig(pieces, "pieces")
        splits, plane = pieces.shape[0], x.numel()
    if rows is not None:
        _ints(rows, "rows")
        if rows.numel() != R:
            raise KernelError("add_rmsnorm: one output row per entry of rows")
        write_x = False
    elif x.shape[0] != R:
        raise KernelError("add_rmsnorm: out must have x's rows")
    _check(core().tl_add_rmsnorm(_ptr(x), _ptr(r), _ptr(w), dtype_code(w.dtype), _ptr(out), dtype_code(out.dtype),
                                 _ptr(rows), R, H, float(eps), int(write_x), _ptr(pieces), splits, plane, _stream()),
           "add_rmsnorm")


def silu_mul(gu: torch.Tensor, out: torch.Tensor, block: int | None = None) -> None:
    """out = silu(gate) * up from gu [T, 2I].  block None: gate = gu[:, :I], up = gu[:, I:]; else gate
    and up columns alternate in blocks of `block` columns (gate first), as a product against weight rows
    interleaved that way leaves them."""
    T, I = out.shape
    if gu.shape != (T, 2 * I) or gu.dtype != out.dtype:
        raise KernelError("silu_mul: gu must be [T, 2I] of out's type")
    blk = I if block is None else int(block)
    if blk <= 0 or I % blk:
        raise KernelError(f"silu_mul: the block of {blk} columns must divide I = {I}")
    _contig(gu, "gu"); _contig(out, "out")
    _check(core().tl_silu_mul(_ptr(gu), _ptr(out), dtype_code(out.dtype), T, I, blk, _stream()), "silu_mul")


def rope_kv_write(qkv: torch.Tensor, bias: torch.Tensor | None, pos: torch.Tensor, req_slot: torch.Tensor,
                  table: torch.Tensor, page_size: int, inv_freq: torch.Tensor, rot: int, nq: int, nkv: int,
                  d: int, k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, write_kv: bool = True,
                  pieces: torch.Tensor | None = None, pairing: str = "half", q_norm: torch.Tensor | None = None,
                  k_norm: torch.Tensor | None = None, norm_eps: float = 0.0) -> None:
    """Bias, rotary encoding of q and k in place, and the write of k, v into their pages.
    `pairing`: "half" rotates dimensions (i, i + rot/2), "interleaved" (2i, 2i + 1).  `q_norm`, `k_norm`
    (float32 [d], both or neither): every q and k head is RMS-normalised over its d dimensions (after the
    bias, before the rotation; statistics in float32) and multiplied by the weight.
    `pieces` [S, T, width] float32: the projection as a split-K product left it; the kernel sums them
    (bfloat16, full rotary, d % 16 == 0 only) and qkv is output only (its q columns are written)."""
    T = qkv.shape[0]
    splits = plane = 0
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"rope_kv_write: pairing {pairing!r} is neither 'half' nor 'interleaved'")
    if (q_norm is None) != (k_norm is None):
        raise KernelError("rope_kv_write: q_norm and k_norm come together")
    for name, w in (("q_norm", q_norm), ("k_norm", k_norm)):
        if w is not None and (w.dtype != torch.float32 or w.numel() != d or not w.is_contiguous()):
            raise KernelError(f"rope_kv_write: {name} must be float32 [d]")
    if pieces is not None and (pairing != "half" or q_norm is not None):
        raise KernelError("rope_kv_write: pieces go with rotate-half pairing and no q/k norm")
    if pieces is not None:
        if (pieces.dtype != torch.float32 or pieces.dim() != 3 or pieces.shape[1:] != qkv.shape
                or qkv.dtype != torch.bfloat16 or rot != d or d % 16):
            raise KernelError("rope_kv_write: pieces must be float32 [S, T, width] for bfloat16 qkv, full rotary, d % 16 == 0")
        _contig(pieces, "pieces")
        splits, plane = pieces.shape[0], qkv.numel()
    if qkv.shape[1] != (nq + 2 * nkv) * d:
        raise KernelError("rope_kv_write: qkv must be [T, (nq + 2 nkv) d]")
    _contig(qkv, "qkv"); _ints(pos, "pos"); _ints(req_slot, "req_slot"); _ints(table, "table")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != rot // 2:
        raise KernelError("rope_kv_write: inv_freq must be float32 [rot/2]")
    if write_kv:
        for name, pages in (("k_pages", k_pages), ("v_pages", v_pages)):
            if pages is None or pages.dtype != qkv.dtype or tuple(pages.shape[1:]) != (nkv, page_size, d):
                raise KernelError(f"rope_kv_write: {name} must be [pages, nkv, page, d] of qkv's type")
            _contig(pages, name)
    _check(core().tl_rope_kv_write(
        _ptr(qkv), dtype_code(qkv.dtype), _ptr(bias), dtype_code(bias.dtype) if bias is not None else 0,
        _ptr(pos), _ptr(req_slot), _ptr(table), table.shape[1], page_size, _ptr(inv_freq), rot, nq, nkv, d,
        _ptr(k_pages) if write_kv else None, _ptr(v_pages) if write_kv else None, int(write_kv), T,
        _ptr(pieces), splits, plane, int(pairing == "interleaved"), _ptr(q_norm), _ptr(k_norm), float(norm_eps),
        table.shape[0], k_pages.shape[0] if write_kv else 0, fault_words(qkv.device), _stream()), "rope_kv_write")


def attn_tokenwise(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                   table: torch.Tensor, page_size: int, pos: torch.Tensor, req_slot: torch.Tensor,
                   nq: int, nkv: int, d: int, window: int | None, scale: float) -> None:
    """Exact-order paged attention; q rows `q_stride` elements apart, out [T, nq*d]."""
    T = out.shape[0]
    if out.shape[1] != nq * d or out.dtype != q.dtype or k_pages.dtype != q.dtype:
        raise KernelError("attn_tokenwise: out must be [T, nq*d] and all tensors of one type")
    if d > 512:
        raise KernelError(f"attn_tokenwise: head_dim {d} > 512 is not supported")
    _contig(out, "out"); _contig(k_pages, "k_pages"); _contig(v_pages, "v_pages")
    _ints(pos, "pos"); _ints(req_slot, "req_slot"); _ints(table, "table")
    _check(core().tl_attn_tokenwise(_ptr(q), q_stride, _ptr(out), dtype_code(q.dtype), _ptr(k_pages), _ptr(v_pages),
                                    _ptr(table), table.shape[1], page_size, _ptr(pos), _ptr(req_slot), T, nq, nkv, d,
                                    int(window or 0), float(scale), table.shape[0], k_pages.shape[0], fault_words(out.device),
                                    _stream()), "attn_tokenwise")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> None:
    """out[M, N] = a[M, K] w[N, K]^T (+ bias), float32 FFMA; w float32 or bfloat16 (widened)."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.float32 or out.dtype != torch.float32 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError("gemm_f32: a [M,K] and out [M,N] must be float32, w [N,K]")
    if a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_f32: a and out must have unit inner stride")
    _contig(w, "w")
    if bias is not None and bias.dtype != w.dtype:
        raise KernelError("gemm_f32: bias must have w's type")
    _check(core().tl_gemm_f32(_ptr(a), a.stride(0), _ptr(w), K, dtype_code(w.dtype), _ptr(bias), _ptr(out),
                              out.stride(0), M, N, K, _stream()), "gemm_f32")


ARGMAX_SLICES = 32


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the largest logit of row r, the lowest index on a tie."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 with unit inner stride")
    _ints(out, "out")
    wide = V >= 8192                                     # wide rows are cut into slices, merged by a second kernel
    partial = torch.empty(R * 2 * ARGMAX_SLICES, dtype=torch.int32, device=logits.device) if wide else None
    _check(core().tl_argmax(_ptr(logits), logits.stride(0), R, V, _ptr(out), _ptr(partial), _stream()), "argmax",
           launches=2 if wide else 1)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, uniform: torch.Tensor,
           out: torch.Tensor) -> None:
    """Per row: temperature <= 0 gives the argmax, else a draw from softmax(logits / T) cut to
    the top-p nucleus, picked by inverse CDF at `uniform`."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with unit inner stride")
    for name, t in (("temperature", temperature), ("top_p", top_p), ("uniform", uniform)):
        if t.dtype != torch.float32 or t.numel() != R:
            raise KernelError(f"sample: {name} must be float32 [R]")
    _ints(out, "out")
    _check(core().tl_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_p), _ptr(uniform),
                            _ptr(out), _stream()), "sample")

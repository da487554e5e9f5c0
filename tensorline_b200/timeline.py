"""The time line of a captured decode step, from stamps the kernels leave themselves.

The tracing build of the libraries (`TENSORLINE_B200_TRACE=1`, see `csrc/common.cuh`) makes the kernels that wait on the
kernel in front of them - the few-token product and the TMA decode attention - write global-timer stamps, eight a block:
block start, dependency wait returned, first and last operand tile landed, block end, and three of their own.  A CUDA
graph keeps the buffer and the slot of each launch, so after some replays the buffer holds the last step: for every
kernel when its blocks started, between which moments its operands streamed in, and when it ended; and between two
kernels how long nothing streamed.  ncu cannot show this (it serialises the launches); the stamps cost a few stores.

    TENSORLINE_B200_TRACE=1 python bench.py --timeline --layers 6            # prints the table of one decode step
"""
from __future__ import annotations

import ctypes

import torch

from .csrc.build import TRACE_BUILD

BLOCKS, STAMPS = 512, 8            # as in csrc/common.cuh


class Timeline:
    """Buffers for the stamps of the libraries named in `libs` ({label: ctypes library}); every launch of theirs from
    now on takes a slot."""

    def __init__(self, libs: dict, device, slots: int = 2048):
        if not TRACE_BUILD:
            raise RuntimeError("the time line needs the tracing build of the kernels: set TENSORLINE_B200_TRACE=1 "
                               "before the package is imported")
        self.slots, self.libs, self.bufs = slots, libs, {}
        for label, lib in libs.items():
            lib.tl_trace_set.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
            lib.tl_trace_set.restype = ctypes.c_int
            lib.tl_trace_build.restype = ctypes.c_int
            if not lib.tl_trace_build():
                raise RuntimeError(f"the {label} library was not compiled with -DTL_TRACE=1")
            buf = torch.zeros(slots * BLOCKS * STAMPS, dtype=torch.int64, device=device)
            lib.tl_trace_set(buf.data_ptr(), slots, 0)
            self.bufs[label] = buf

    def stop(self) -> None:
        for lib in self.libs.values():
            lib.tl_trace_set(None, 0, 0)

    def last_step(self, step_ms: float) -> list:
        """[(label, stamps [blocks, 8] int64 nanoseconds from the step's first block start)] of the kernels whose blocks
        started within the last `step_ms` milliseconds of what was recorded, in order of their first block."""
        torch.cuda.synchronize()
        recs = []
        for label, buf in self.bufs.items():
            t = buf.view(self.slots, BLOCKS, STAMPS).cpu()
            for s in range(self.slots):
                live = t[s][:, 0] != 0
                if bool(live.any()):
                    recs.append((label, t[s][live]))
        if not recs:
            return []
        end = max(int(b[:, 4].max()) for _, b in recs)
        last = [(n, b) for n, b in recs if int(b[:, 0].min()) > end - int(step_ms * 1e6 * 0.98)]
        last.sort(key=lambda r: int(r[1][:, 0].min()))
        t0 = int(last[0][1][:, 0].min())
        return [(n, b - t0) for n, b in last]


def table(kernels: list) -> str:
    """One line a kernel (microseconds from the step's first block): when its blocks started, when the first and the last
    operand tile had landed, when its blocks ended, and how long nothing streamed since the kernel before."""
    def us(x):
        return float(x) / 1e3

    lines = ["kernel  blocks   starts             wait done   first tile   last tile   ends               no stream before"]
    prev_last = None
    for label, b in kernels:
        first = b[:, 2][b[:, 2] > 0]
        last = b[:, 3][b[:, 3] > 0]
        wait = b[:, 1][b[:, 1] > 0]
        f_min = us(first.min()) if first.numel() else float("nan")
        l_max = us(last.max()) if last.numel() else float("nan")
        gap = "" if prev_last is None else f"{f_min - prev_last:+6.2f}"
        lines.append(f"{label:7s} {b.shape[0]:5d}   {us(b[:, 0].min()):7.2f}..{us(b[:, 0].max()):7.2f}   "
                     f"{us(wait.median()) if wait.numel() else float('nan'):8.2f}   {f_min:9.2f}   {l_max:9.2f}   "
                     f"{us(b[:, 4].min()):7.2f}..{us(b[:, 4].max()):7.2f}   {gap}")
        prev_last = l_max
        d = b.double()
        if label.startswith("attn"):
            if not bool((b[:, 7] > 0).any()):               # no cluster: the ranges' parts go to a combine kernel
                continue
            m = lambda x: f"{float(x.median()) / 1e3:.2f}"
            lines.append(f"          a block (medians): wait -> first product {m(d[:, 2] - d[:, 1])}, last stage -> worked through "
                         f"{m(d[:, 5] - d[:, 3])}, -> parts combined {m(d[:, 6] - d[:, 5])}, cluster barrier {m(d[:, 7] - d[:, 6])}, "
                         f"merge and store {m(d[:, 4] - d[:, 7])}")
        if not label.startswith("attn") and bool((b[:, 5] > 0).any()):
            m = lambda x: f"{float(x.median()) / 1e3:.2f}"
            lines.append(f"          a block (medians, normed operand): wait -> rstd known {m(d[:, 5] - d[:, 1])}, -> raw tile landed "
                         f"{m(d[:, 6] - d[:, 1])}, -> operand tile made {m(d[:, 7] - d[:, 1])}, -> first product {m(d[:, 2] - d[:, 1])}")
    return "\n".join(lines)

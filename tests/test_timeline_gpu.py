"""The tracing build of the kernels (TENSORLINE_B200_TRACE=1): the stamps a product and a decode attention launch leave,
read back through `tensorline_b200.timeline`.  Run in a process of its own, because the build is chosen at import."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

SCRIPT = r"""
import torch
from tensorline_b200 import ops_attention, ops_gemm, timeline
dev = torch.device("cuda", 0)
d, nq, nkv, ps, n = 64, 8, 2, 16, 700
tl = timeline.Timeline({"product": ops_gemm.lib(), "attn": ops_attention.attn_lib(d)}, dev, slots=16)
g = torch.Generator().manual_seed(0)
x = (torch.randn(8, 1024, generator=g) * 0.5).to(torch.bfloat16).to(dev)
w = (torch.randn(512, 1024, generator=g) * 0.05).to(torch.bfloat16).to(dev)
y = ops_gemm.gemm_tc(x, w)
assert float((y.float().cpu() - x.float().cpu() @ w.float().cpu().T).abs().max()) < 0.1     # the stamps change no result
pages = n // ps + 2
kp = torch.randn(pages + 1, nkv, ps, d, generator=g).to(torch.bfloat16).to(dev)
vp = torch.randn(pages + 1, nkv, ps, d, generator=g).to(torch.bfloat16).to(dev)
table = torch.arange(pages, dtype=torch.int32).reshape(1, pages).to(dev)
q = torch.randn(1, nq * d, generator=g).to(torch.bfloat16).to(dev)
out = torch.zeros(1, nq * d, dtype=torch.bfloat16, device=dev)
i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
ops_attention.decode(q, nq * d, out, kp, vp, table, ps, i32([0]), i32([n - 1]), i32([0]), 1, nq, nkv, d, None, d ** -0.5,
                     256, 3, None, None, tma=True, cluster=True)
ops_gemm.check_status()
tl.stop()
kernels = tl.last_step(1e6)
assert [k for k, _ in kernels] == ["product", "attn"], [k for k, _ in kernels]
prod, attn = kernels[0][1], kernels[1][1]
assert prod.shape[0] >= 4 and attn.shape == (3 * nkv, 8)
for b in prod.tolist():                                   # start <= wait done <= first stage <= last stage <= end
    assert 0 <= b[0] <= b[1] <= b[2] <= b[3] <= b[4], b
for b in attn.tolist():                                   # ... <= last stage worked through <= cluster barrier <= end
    assert 0 <= b[0] <= b[1] and b[0] <= b[2] <= b[3] <= b[5] <= b[6] <= b[7] <= b[4], b
print(timeline.table(kernels))
print("timeline ok")
"""


def test_kernels_of_the_tracing_build_leave_their_stamps():
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, TENSORLINE_B200_TRACE="1", PYTHONPATH=str(root))
    p = subprocess.run([sys.executable, "-c", SCRIPT], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "timeline ok" in p.stdout, p.stdout[-2000:] + p.stderr[-4000:]
    assert "no stream before" in p.stdout


def test_the_ordinary_build_records_nothing():
    import ctypes
    import torch
    from tensorline_b200 import ops_gemm
    lib = ops_gemm.lib()
    lib.tl_trace_set.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    lib.tl_trace_build.restype = ctypes.c_int
    if lib.tl_trace_build():
        pytest.skip("this process runs the tracing build")
    buf = torch.zeros(4 * 512 * 8, dtype=torch.int64, device="cuda")
    lib.tl_trace_set(buf.data_ptr(), 4, 0)
    x = torch.randn(8, 1024, device="cuda").to(torch.bfloat16)
    w = torch.randn(256, 1024, device="cuda").to(torch.bfloat16)
    ops_gemm.gemm_tc(x, w)
    lib.tl_trace_set(None, 0, 0)
    torch.cuda.synchronize()
    assert int(buf.abs().sum()) == 0

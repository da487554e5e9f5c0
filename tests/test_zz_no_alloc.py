"""The decode-attention entry point that allocates nothing (`tl_attn_decode_static`, declared in
tensorline_b200/csrc/attn_static.h) against the ordinary entry point.

Some users of the library cannot call cudaMalloc where they call the kernel: they run inside another
runtime's memory plan, or on a path where an allocation may block, or they are C programs without an
allocator.  For them the scratch of the split-KV kernel is a fixed array inside the library.  This
test calls that entry point through its exported C symbol, twice in a row with different shapes (the
array keeps the first call's contents, which the second call must not see), and compares its output
with the ordinary entry point's, which gets torch-allocated scratch, and with the attention formula
written out in float64.  It also checks that a request beyond the array's size is refused with a
message, and a context that ends exactly at chunk * splits.  The file name makes pytest collect it last.
"""
import ctypes

import pytest
import torch

from tests.gpu_helpers import BF16, assert_close, i32, table_tensor

pytestmark = pytest.mark.gpu

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _setup(B, ctx_lens, nq, nkv, d, ps, seed):
    g = torch.Generator().manual_seed(seed)
    num_pages, max_pages = 400, 128
    kp = torch.randn(num_pages + 1, nkv, ps, d, generator=g).to(torch.bfloat16).cuda()
    vp = torch.randn(num_pages + 1, nkv, ps, d, generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(num_pages, generator=g).tolist()
    rows, used = [], 0
    for n in ctx_lens:
        need = -(-(n + 1) // ps)
        rows.append(perm[used:used + need])
        used += need
    q = (torch.randn(B, nq * d, generator=g) * 2).to(torch.bfloat16).cuda()
    return q, kp, vp, table_tensor(rows, max_pages, num_pages), num_pages


def _plain_rows(q, kp, vp, table, ps, ctx_lens, nq, nkv, d):
    """softmax(q k^T / sqrt(d)) v over the keys 0..ctx_len of each request, float64 (tensorline/paged_attn.py:33-57)."""
    out = torch.zeros(len(ctx_lens), nq * d, dtype=torch.float64)
    qf, kf, vf, tab = q.double().cpu(), kp.double().cpu(), vp.double().cpu(), table.cpu()
    for b, last in enumerate(ctx_lens):
        pos = torch.arange(last + 1)
        pages, offs = tab[b, pos // ps].long(), pos % ps
        for h in range(nq):
            kh = h // (nq // nkv)
            k, v = kf[pages, kh, offs], vf[pages, kh, offs]
            s = (k @ qf[b, h * d:(h + 1) * d]) * d ** -0.5
            out[b, h * d:(h + 1) * d] = torch.softmax(s, 0) @ v
    return out


def _static_call(lib, q, out, kp, vp, table, ps, B, ctx_lens, nq, nkv, d, chunk, splits):
    fn = lib.tl_attn_decode_static
    fn.argtypes = [_P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, ctypes.c_char_p, _I]
    fn.restype = ctypes.c_int
    q_start, start_pos, slots = i32(list(range(B + 1))), i32(ctx_lens), i32(list(range(B)))
    err = ctypes.create_string_buffer(512)
    rc = fn(q.data_ptr(), q.shape[1], out.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.shape[1], ps,
            q_start.data_ptr(), start_pos.data_ptr(), slots.data_ptr(), B, nq, nkv, 0, d ** -0.5, chunk, splits,
            torch.cuda.current_stream().cuda_stream, err, 512)
    torch.cuda.synchronize()
    return rc, err.value.decode()


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from tensorline_b200 import ops_attention
    nq, nkv, d, ps = 14, 2, 64, 16
    lib = ops_attention.attn_lib(d)
    # two calls in a row: many ranges first, then fewer requests and ranges over stale partials
    for B, ctx_lens, chunk, splits, seed in ((5, [700, 63, 64, 1, 333], 128, 6, 1), (2, [250, 40], 64, 4, 2)):
        q, kp, vp, table, _ = _setup(B, ctx_lens, nq, nkv, d, ps, seed)
        want = torch.zeros(B, nq * d, dtype=torch.bfloat16, device="cuda")
        po = torch.empty(B, nq, splits, d, device="cuda")
        pml = torch.empty(B, nq, splits, 2, device="cuda")
        ops_attention.decode(q, nq * d, want, kp, vp, table, ps, i32(list(range(B + 1))), i32(ctx_lens),
                             i32(list(range(B))), B, nq, nkv, d, None, d ** -0.5, chunk, splits, po, pml, tma=False)
        got = torch.zeros_like(want)
        rc, msg = _static_call(lib, q, got, kp, vp, table, ps, B, ctx_lens, nq, nkv, d, chunk, splits)
        assert rc == 0, msg
        assert float(want.float().abs().max()) > 0.1
        assert_close(got, want, f"static scratch, B={B}", **BF16)
        assert_close(got, _plain_rows(q, kp, vp, table, ps, ctx_lens, nq, nkv, d), f"static scratch against the formula, B={B}", **BF16)
    # one range per request needs no scratch at all
    q, kp, vp, table, _ = _setup(2, [100, 30], nq, nkv, d, ps, 3)
    want, got = (torch.zeros(2, nq * d, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    ops_attention.decode(q, nq * d, want, kp, vp, table, ps, i32([0, 1, 2]), i32([100, 30]), i32([0, 1]), 2, nq, nkv, d,
                         None, d ** -0.5, 128, 1, tma=False)
    rc, msg = _static_call(lib, q, got, kp, vp, table, ps, 2, [100, 30], nq, nkv, d, 128, 1)
    assert rc == 0, msg
    assert_close(got, want, "static scratch, one range", **BF16)
    assert_close(got, _plain_rows(q, kp, vp, table, ps, [100, 30], nq, nkv, d), "static scratch against the formula, one range", **BF16)
    # the key ranges must cover the longest context: one that ends exactly at chunk * splits is read to its last key
    q, kp, vp, table, _ = _setup(2, [255, 17], nq, nkv, d, ps, 5)
    got = torch.zeros(2, nq * d, dtype=torch.bfloat16, device="cuda")
    rc, msg = _static_call(lib, q, got, kp, vp, table, ps, 2, [255, 17], nq, nkv, d, 64, 4)       # 4 ranges of 64 = 256 keys
    assert rc == 0, msg
    assert_close(got, _plain_rows(q, kp, vp, table, ps, [255, 17], nq, nkv, d), "context ending at chunk * splits", **BF16)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from tensorline_b200 import ops_attention
    nq, nkv, d, ps = 14, 2, 64, 16
    lib = ops_attention.attn_lib(d)
    q, kp, vp, table, _ = _setup(2, [100, 30], nq, nkv, d, ps, 4)
    out = torch.full((2, nq * d), 7.0, dtype=torch.bfloat16, device="cuda")
    B_claimed = 4000                                     # 4000 * 14 * 32 * 66 floats is far beyond 1 Mi floats
    fn = lib.tl_attn_decode_static
    fn.argtypes = [_P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, ctypes.c_char_p, _I]
    fn.restype = ctypes.c_int
    err = ctypes.create_string_buffer(512)
    rc = fn(q.data_ptr(), q.shape[1], out.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.shape[1], ps,
            None, None, None, B_claimed, nq, nkv, 0, 0.125, 64, 32, torch.cuda.current_stream().cuda_stream, err, 512)
    assert rc != 0 and "exceed the static scratch" in err.value.decode()
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                      # nothing was launched
    rc, msg = _static_call(lib, q, out, kp, vp, table, ps, 2, [100, 30], nq, nkv, d, 100, 2)
    assert rc != 0 and "multiple of 64" in msg

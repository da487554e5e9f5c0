"""Each CUDA kernel alone against its plain reference, at sizes that are not the engine's."""
import math

import pytest
import torch

from tests.gpu_helpers import BF16, F32, assert_close, i32, scatter_pages, table_tensor
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def tol(dt):
    return F32 if dt == torch.float32 else BF16


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("wdt", DT)
def test_embedding(wdt):
    from tensorline_b200 import ops
    table = rnd(53, 24, seed=1, dtype=wdt)
    ids = [0, 52, 7, 7, 31]
    x = torch.empty(5, 24, dtype=torch.float32, device="cuda")
    ops.embed(x, table.cuda(), i32(ids))
    assert torch.equal(x.cpu().double(), plain.embedding(table.double(), ids))


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("wdt", DT)
@pytest.mark.parametrize("H", [100, 3, 1030])
def test_add_rmsnorm(adt, wdt, H):
    from tensorline_b200 import ops
    T, eps = 7, 3e-5
    x = rnd(T, H, seed=2, scale=3.0)
    r = rnd(T, H, seed=3, dtype=adt)
    w = (1 + rnd(H, seed=4, scale=0.3)).to(wdt)
    xd, out = x.cuda(), torch.empty(T, H, dtype=adt, device="cuda")
    ops.add_rmsnorm(xd, r.cuda(), w.cuda(), out, eps)
    want_x = x.double() + r.double()
    assert_close(xd, want_x, "residual sum", rtol=1e-6, atol=1e-6)            # a float32 sum
    assert_close(out, plain.rms_norm(want_x, w.double(), eps), "norm", **tol(adt))
    # without a residual, x stays as it is; with row selection too
    xd2 = x.cuda()
    ops.add_rmsnorm(xd2, None, w.cuda(), out, eps)
    assert torch.equal(xd2.cpu(), x)
    assert_close(out, plain.rms_norm(x.double(), w.double(), eps), "norm only", **tol(adt))
    rows = [5, 0, 5]
    out3 = torch.empty(3, H, dtype=adt, device="cuda")
    xd3 = x.cuda()
    ops.add_rmsnorm(xd3, r.cuda(), w.cuda(), out3, eps, rows=i32(rows))
    assert torch.equal(xd3.cpu(), x)
    assert_close(out3, plain.rms_norm(want_x[rows], w.double(), eps), "selected rows", **tol(adt))


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("I", [37, 40])
def test_silu_mul(adt, I):
    from tensorline_b200 import ops
    T = 5
    gu = rnd(T, 2 * I, seed=5, scale=3.0, dtype=adt)
    out = torch.empty(T, I, dtype=adt, device="cuda")
    ops.silu_mul(gu.cuda(), out)
    g, u = gu[:, :I].double(), gu[:, I:].double()
    assert_close(out, g / (1 + torch.exp(-g)) * u, "silu*up", **tol(adt))


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("I,block", [(48, 8), (192, 64), (35, 5)])
def test_silu_mul_interleaved(adt, I, block):
    """Gate and up columns alternating in blocks give what the plain layout gives."""
    from tensorline_b200 import ops
    T = 3
    gu = rnd(T, 2 * I, seed=6, scale=3.0, dtype=adt)
    mixed = torch.stack((gu[:, :I].view(T, I // block, block), gu[:, I:].view(T, I // block, block)), dim=2).reshape(T, 2 * I)
    a = torch.empty(T, I, dtype=adt, device="cuda")
    b = torch.empty_like(a)
    ops.silu_mul(gu.cuda(), a)
    ops.silu_mul(mixed.contiguous().cuda(), b, block=block)
    assert torch.equal(a, b)
    with pytest.raises(ops.KernelError, match="divide"):
        ops.silu_mul(gu.cuda(), a, block=I - 1)


@pytest.mark.parametrize("T", [1, 8, 37, 64])
def test_tcgen05_product_with_the_activation_in_its_epilogue(T):
    """Against interleaved gate / up rows the gated epilogue gives bit for bit what the product, stored in
    bfloat16, followed by the activation kernel gives."""
    from tensorline_b200 import ops, ops_gemm
    I, K = 320, 520
    x = rnd(T, K, seed=1, dtype=torch.bfloat16).cuda()
    w = rnd(2 * I, K, seed=2, scale=0.1, dtype=torch.bfloat16).cuda()          # rows already in blocks of 64 + 64
    assert not ops_gemm.can_gate(T, 2 * I + 64, K) and not ops_gemm.can_gate(300, 2 * I, K)
    kw = dict(swap=1, bn=16 if T <= 16 else 64, splits=1)
    gu = ops_gemm.gemm_tc(x, w, **kw)
    want = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
    ops.silu_mul(gu, want, block=64)
    got = ops_gemm.gemm_tc(x, w, gated=True, **kw)
    ops_gemm.check_status()
    assert got.shape == (T, I) and torch.equal(got, want)
    full = (x.double() @ w.double().T).view(T, I // 64, 2, 64)
    g, u = full[:, :, 0].reshape(T, I), full[:, :, 1].reshape(T, I)
    assert_close(got, g / (1 + torch.exp(-g)) * u, "silu(gate) * up", rtol=3e-2, atol=3e-2)
    with pytest.raises(ops.KernelError, match="gated"):
        ops_gemm.gemm_tc(x, w, gated=True, swap=1, bn=16, splits=2)


@pytest.mark.parametrize("wdt", DT)
def test_gemm_f32_exact_order(wdt):
    from tensorline_b200 import ops
    M, N, K = 37, 70, 45
    a, w = rnd(M, K, seed=6), rnd(N, K, seed=7, dtype=wdt)
    out = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.gemm_f32(a.cuda(), w.cuda(), out)
    assert_close(out, a.double() @ w.double().T, "gemm", **F32)
    # a row's result does not depend on the other rows of the launch
    one = torch.empty(1, N, dtype=torch.float32, device="cuda")
    ops.gemm_f32(a[17:18].cuda(), w.cuda(), one)
    assert torch.equal(one[0], out[17])


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("rot", [None, 8])
@pytest.mark.parametrize("d", [24, 32])
def test_rope_and_kv_write(adt, rot, d):
    from tensorline_b200 import ops
    nq, nkv, ps, theta = 3, 2, 4, 5000.0
    rdim = d if rot is None else rot
    pos = [0, 1, 2, 9, 10, 4097]
    slots = [1, 1, 1, 0, 0, 2]
    T = len(pos)
    qkv = rnd(T, (nq + 2 * nkv) * d, seed=8, dtype=adt)
    bias = rnd((nq + 2 * nkv) * d, seed=9, scale=0.5, dtype=adt)
    max_pages, num_pages = 1100, 3400
    g = torch.Generator().manual_seed(3)
    table = torch.randperm(num_pages, generator=g)[:3 * max_pages].reshape(3, max_pages).to(torch.int32)
    kp = torch.zeros(num_pages + 1, nkv, ps, d, dtype=adt, device="cuda")
    vp = torch.zeros_like(kp)
    inv_freq = (theta ** (-torch.arange(0, rdim, 2, dtype=torch.float64) / rdim)).float()
    q = qkv.cuda()
    ops.rope_kv_write(q, bias.cuda(), i32(pos), i32(slots), table.cuda(), ps, inv_freq.cuda(), rdim, nq, nkv, d, kp, vp)
    x = (qkv.double() + bias.double()).view(T, nq + 2 * nkv, d)
    cos, sin = plain.rope_cos_sin(pos, rdim, theta)
    rotated = torch.cat((plain.apply_rope(x[..., :rdim], cos, sin), x[..., rdim:]), dim=-1)
    assert_close(q.view(T, -1, d)[:, :nq], rotated[:, :nq], "q", **tol(adt))
    for t in range(T):
        page, off = int(table[slots[t], pos[t] // ps]), pos[t] % ps
        assert_close(kp[page, :, off], rotated[t, nq:nq + nkv], f"k of token {t}", **tol(adt))
        assert_close(vp[page, :, off], x[t, nq + nkv:], f"v of token {t}", **tol(adt))
    assert int((kp != 0).any(dim=-1).sum()) == T * nkv                       # nothing else was written


def test_rope_sums_the_pieces_of_a_split_product():
    """Handed the unsummed float32 pieces of the projection, the rotary kernel gives bit for bit what it
    gives from their bfloat16 sum: q in the qkv buffer, k and v in the pages."""
    from tensorline_b200 import ops
    nq, nkv, d, ps, S = 5, 2, 32, 8, 3
    pos, slots = [0, 7, 8, 300], [1, 0, 0, 1]
    T, W = len(pos), (5 + 2 * 2) * 32
    pieces = rnd(S, T, W, seed=21).cuda()
    whole = (pieces[0] + pieces[1] + pieces[2]).to(torch.bfloat16)
    bias = rnd(W, seed=22, scale=0.5, dtype=torch.bfloat16).cuda()
    table = torch.randperm(90, generator=torch.Generator().manual_seed(4))[:80].reshape(2, 40).to(torch.int32).cuda()
    inv_freq = (10000.0 ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)).float().cuda()
    outs = []
    for use_pieces in (False, True):
        kp = torch.zeros(91, nkv, ps, d, dtype=torch.bfloat16, device="cuda")
        vp = torch.zeros_like(kp)
        qkv = torch.full((T, W), 7.0, dtype=torch.bfloat16, device="cuda") if use_pieces else whole.clone()
        ops.rope_kv_write(qkv, bias, i32(pos), i32(slots), table, ps, inv_freq, d, nq, nkv, d, kp, vp,
                          pieces=pieces if use_pieces else None)
        outs.append((qkv[:, :nq * d].clone(), kp, vp))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert float(outs[0][1].abs().sum()) > 0
    with pytest.raises(ops.KernelError, match="pieces"):
        ops.rope_kv_write(whole.float(), bias.float(), i32(pos), i32(slots), table, ps, inv_freq, d, nq, nkv, d,
                          outs[0][1].float(), outs[0][2].float(), pieces=pieces)


@pytest.mark.parametrize("V", [5003, 40007])            # one block per row; slices merged by a second kernel
def test_argmax_lowest_index_wins(V):
    from tensorline_b200 import ops
    logits = rnd(6, V, seed=10)
    logits[2, 4000] = logits[2, 17] = 50.0
    logits[3, V - 1] = 60.0
    logits[4, 0] = 60.0
    logits[5, V // 2 + 3] = logits[5, V - 5] = 70.0
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.argmax(logits.cuda(), out)
    want = logits.argmax(-1).tolist()
    want[2], want[5] = 17, V // 2 + 3
    assert out.tolist() == want


@pytest.mark.parametrize("V,R", [(1237, 64), (5003, 9), (40007, 24)])       # clusters of 1, 2 and 8 blocks a row
@pytest.mark.parametrize("top_p", [1.0, 0.7, 0.2])
def test_sampling_matches_reference_distribution(top_p, V, R):
    """The picked token is the one the plain inverse-CDF picks for the same uniform number; the kept
    set is the reference's nucleus."""
    from tensorline_b200 import ops
    logits = rnd(R, V, seed=11, scale=2.5)
    logits[0, V - 3] = 9.0                                                  # most of row 0's mass at the far end
    logits[1] *= 0.01                                                       # nearly flat: a nucleus of thousands
    temps = torch.full((R,), 0.8)
    temps[5] = 0.0                                                          # a greedy row among sampled ones
    logits[5, V - 2] = logits[5, 3] = 11.0                                  # whose maximum is tied across slices
    g = torch.Generator().manual_seed(12)
    u = torch.rand(R, generator=g)
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(logits.cuda(), temps.cuda(), torch.full((R,), top_p).cuda(), u.cuda(), out)
    got = out.tolist()
    for r in range(R):
        if temps[r] <= 0:
            assert got[r] == 3
            continue
        probs = plain.sampling_distribution(logits[r], float(temps[r]), top_p)
        assert probs[got[r]] > 0, f"row {r}: token {got[r]} is outside the nucleus"
        cdf = torch.cumsum(probs, 0)
        lo = float(cdf[got[r]] - probs[got[r]])
        assert lo - 1e-5 <= float(u[r]) <= float(cdf[got[r]]) + 1e-5, f"row {r}: u={float(u[r])} not in the token's interval"


def _plain_attention_rows(q, k, v, pos_q, window):
    """q [n, nq, d] at positions pos_q over the whole k, v [len, nkv, d]."""
    n, nq, d = q.shape
    g = nq // k.shape[1]
    out = torch.empty_like(q)
    for i, p in enumerate(pos_q):
        lo = max(0, p - window + 1) if window else 0
        for h in range(nq):
            s = (k[lo:p + 1, h // g] @ q[i, h]) * d ** -0.5
            out[i, h] = torch.softmax(s, 0) @ v[lo:p + 1, h // g]
    return out


ATT_CASES = [  # nq, nkv, d, page, context lengths before the step, tokens in the step, window
    (4, 2, 16, 4, [0, 5, 31], [9, 1, 2], None),
    (3, 1, 32, 8, [0, 130], [70, 3], 24),
    (7, 1, 128, 16, [300, 0, 65], [1, 1, 1], None),
    (6, 2, 48, 16, [63, 64, 1399], [1, 1, 1], None),
    (14, 2, 64, 64, [15, 0], [17, 200], 100),
    (20, 1, 16, 2, [77], [1], None),
    (5, 5, 80, 32, [257], [1], 33),
    (28, 4, 128, 16, [0, 130, 700], [300, 3, 1], None),
    (6, 2, 192, 32, [63, 64], [70, 1], None),
    (4, 4, 256, 64, [257, 0], [1, 150], 33),
    (7, 7, 64, 2, [30], [150], 50),
    (28, 4, 128, 16, [1, 1000, 700, 63], [1, 1, 1, 1], None),
    (8, 2, 64, 8, [500, 129], [1, 1], 200),
    (3, 1, 256, 32, [333], [1], None),
    (7, 1, 128, 16, [0, 700, 41], [200, 37, 90], None),     # several 128-row tiles a request: both tiles of a pair, a lone first tile
    (14, 2, 64, 8, [300], [130], 70),                       # a window that lets the later tile of a pair start further on
    (4, 2, 128, 64, [0], [129], None),
]


@pytest.mark.parametrize("case", ATT_CASES, ids=[f"q{c[0]}kv{c[1]}d{c[2]}p{c[3]}" for c in ATT_CASES])
@pytest.mark.parametrize("kernel", ["exact_f32", "exact_bf16", "mma_bf16", "tcgen05_bf16", "tcgen05_pair_bf16", "tcgen05_p_tmem_bf16", "tcgen05_p_tmem64_bf16", "tcgen05_pair_split_bf16"])
def test_paged_attention(case, kernel):
    """Decode and prefill attention over scattered pages against the plain formula."""
    from tensorline_b200 import ops, ops_attention
    nq, nkv, d, ps, ctx_lens, step_lens, window = case
    if kernel in ("tcgen05_pair_bf16", "tcgen05_p_tmem_bf16", "tcgen05_p_tmem64_bf16", "tcgen05_pair_split_bf16") and d % 64:
        pytest.skip("no tcgen05 build for this head size")
    if kernel == "tcgen05_bf16" and (d % 64 or ps < 2):
        with pytest.raises(ops.KernelError):
            ops_attention.attn_tc_lib(d) if d % 64 else ops_attention.prefill_tc(
                torch.zeros(1, nq * d, dtype=torch.bfloat16, device="cuda"), nq * d, None, None, None,
                torch.zeros(1, 1, dtype=torch.int32, device="cuda"), ps, None, None, None, [0, 1], nq, nkv, d, None, 1.0)
        return
    pair_ok = d <= 128 and d % 64 == 0 and ps >= 8
    adt = torch.float32 if kernel == "exact_f32" else torch.bfloat16
    B = len(ctx_lens)
    max_pages, num_pages = 128, 300
    kps = torch.zeros(num_pages + 1, nkv, ps, d, dtype=adt)
    vps = torch.zeros_like(kps)
    rows, qs, want, pos_all, slot_all = [], [], [], [], []
    used = 0
    for b in range(B):
        n = ctx_lens[b] + step_lens[b]
        k = rnd(n, nkv, d, seed=20 + b, dtype=adt)
        v = rnd(n, nkv, d, seed=40 + b, dtype=adt)
        q = rnd(step_lens[b], nq, d, seed=60 + b, scale=2.0, dtype=adt)
        if b == 0 and n > 40:                       # one far key that must win: a planted score
            k[3] *= 0; k[3, :, 0] = 8.0; q[-1] *= 0; q[-1, :, 0] = 8.0
        need = -(-n // ps)
        g = torch.Generator().manual_seed(100 + b)
        mine = (torch.randperm(num_pages // B, generator=g)[:need] * B + b).tolist()   # interleaved, disjoint
        for i in range(n):
            kps[mine[i // ps], :, i % ps] = k[i]
            vps[mine[i // ps], :, i % ps] = v[i]
        rows.append(mine)
        pq = list(range(ctx_lens[b], n))
        want.append(_plain_attention_rows(q.double(), k.double(), v.double(), pq, window))
        qs.append(q)
        pos_all += pq
        slot_all += [b] * step_lens[b]
    q_all = torch.cat(qs).reshape(-1, nq * d).cuda()
    T = q_all.shape[0]
    out = torch.zeros(T, nq * d, dtype=adt, device="cuda")
    table = table_tensor(rows, max_pages, num_pages)
    kd, vd = kps.cuda(), vps.cuda()
    scale = d ** -0.5
    if kernel in ("tcgen05_bf16", "tcgen05_pair_bf16", "tcgen05_p_tmem_bf16", "tcgen05_p_tmem64_bf16", "tcgen05_pair_split_bf16"):
        import functools
        q_start = [0]
        for n in step_lens:
            q_start.append(q_start[-1] + n)
        fn = ops_attention.prefill_tc if kernel == "tcgen05_bf16" else functools.partial(
            ops_attention.prefill_tc_pair, p_in_tmem={"tcgen05_p_tmem_bf16": True, "tcgen05_p_tmem64_bf16": "64"}.get(kernel, False))
        if kernel == "tcgen05_pair_split_bf16":             # every block's key tiles dealt out to three blocks (some get none)
            fn = functools.partial(ops_attention.prefill_tc_pair, p_in_tmem="64", ksplit=3)
        took = fn(q_all, nq * d, out, kd, vd, table, ps, i32(q_start), i32(ctx_lens), i32(list(range(B))),
                  q_start, nq, nkv, d, window, scale)
        from tensorline_b200 import ops_gemm
        ops_gemm.check_status()
        if kernel != "tcgen05_bf16":
            assert took == pair_ok                                         # other sizes are left to the other kernels
            if not took:
                return
        # the same tiles taken longest first over all requests: every row as before, bit for bit
        order = ops_attention.tile_order(q_start, ctx_lens, nq // nkv, 128 if kernel == "tcgen05_bf16" else 256, "cuda")
        assert (order is None) == (B == 1)
        if order is not None:
            again = torch.zeros_like(out)
            fn(q_all, nq * d, again, kd, vd, table, ps, i32(q_start), i32(ctx_lens), i32(list(range(B))),
               q_start, nq, nkv, d, window, scale, order)
            ops_gemm.check_status()
            assert torch.equal(again, out)
    elif kernel != "mma_bf16":
        ops.attn_tokenwise(q_all, nq * d, out, kd, vd, table, ps, i32(pos_all), i32(slot_all), nq, nkv, d, window, scale)
    else:
        q_start = [0]
        for n in step_lens:
            q_start.append(q_start[-1] + n)
        args = (q_all, nq * d, out, kd, vd, table, ps, i32(q_start), i32(ctx_lens), i32(list(range(B))))
        if all(n == 1 for n in step_lens):
            span = max(c + 1 for c in ctx_lens)
            for splits_wanted in (1, 3, 64):        # one range, a few, and more ranges than tiles
                tiles = -(-span // 64)
                splits = min(splits_wanted, tiles)
                chunk = -(-tiles // splits) * 64
                splits = -(-tiles * 64 // chunk)
                po = torch.full((B, nq, splits, d), float("nan"), device="cuda")
                pml = torch.full((B, nq, splits, 2), float("nan"), device="cuda")
                out.zero_()
                # K, V by cp.async, or by TMA where the sizes allow it; with TMA, the ranges merged by a second
                # kernel or (2..8 ranges, groups of up to 16 heads) inside a thread-block cluster
                for tma, cluster in ((False, False), (True, False), (True, True)):
                    out.zero_()
                    ops_attention.decode(*args, B, nq, nkv, d, window, scale, chunk, splits, po, pml, tma=tma, cluster=cluster)
                    assert_close(out.view(T, nq, d), torch.cat(want), f"decode, {splits} splits, tma {tma}, cluster {cluster}", **BF16)
            out.zero_()
        ops_attention.prefill(*args, q_start, nq, nkv, d, window, scale)
        order = ops_attention.tile_order(q_start, ctx_lens, nq // nkv, 64, "cuda")
        if order is not None:
            again = torch.zeros_like(out)
            ops_attention.prefill(q_all, nq * d, again, *args[3:], q_start, nq, nkv, d, window, scale, order)
            assert torch.equal(again, out)
    assert_close(out.view(T, nq, d), torch.cat(want), kernel, **tol(adt))


@pytest.mark.parametrize("window", [None, 3000])
def test_attention_over_a_long_context(window):
    """9,000 cached tokens (563 pages of 16): a decode step with few and with many key ranges, by cp.async and
    by TMA, and a 300-token portion on top of the cache through every prefill kernel, against the plain
    formula.  One far key is planted so that it must win for the last query."""
    from tensorline_b200 import ops_attention, ops_gemm
    nq, nkv, d, ps, ctx, step = 4, 1, 128, 16, 9000, 300
    n = ctx + step
    k, v = rnd(n, nkv, d, seed=70, dtype=torch.bfloat16), rnd(n, nkv, d, seed=71, dtype=torch.bfloat16)
    q = rnd(step, nq, d, seed=72, scale=2.0, dtype=torch.bfloat16)
    far = 6500 if window else 17                                    # inside the window, or near the start
    k[far] *= 0; k[far, :, 0] = 9.0; q[-1] *= 0; q[-1, :, 0] = 9.0
    num_pages = 700
    kd, vd, order = scatter_pages(k, v, ps, num_pages, seed=5)
    table = table_tensor([order], 640, num_pages)
    scale = d ** -0.5
    rows = [0, 1, 150, step - 2, step - 1]                          # checked against the float64 formula
    want = _plain_attention_rows(q[rows].double(), k.double(), v.double(), [ctx + r for r in rows], window)
    qd = q.reshape(step, nq * d).cuda()
    q_start, pos0, slots = i32([0, step]), i32([ctx]), i32([0])
    outs = {}
    for name, fn in (("mma", ops_attention.prefill), ("tcgen05", ops_attention.prefill_tc), ("pair", ops_attention.prefill_tc_pair)):
        out = torch.zeros(step, nq * d, dtype=torch.bfloat16, device="cuda")
        fn(qd, nq * d, out, kd, vd, table, ps, q_start, pos0, slots, [0, step], nq, nkv, d, window, scale)
        ops_gemm.check_status()
        assert_close(out.view(step, nq, d)[rows], want, f"{name} prefill over a long cache", **BF16)
        outs[name] = out
    # the decode step: the last token alone, all keys before it cached
    last = n - 1
    want1 = _plain_attention_rows(q[-1:].double(), k.double(), v.double(), [last], window)
    q1 = q[-1:].reshape(1, nq * d).cuda()
    tiles = -(-(min(n, window + 63) if window else n) // 64)
    for splits_wanted in (1, 7, 64):
        chunk = -(-tiles // splits_wanted) * 64
        splits = -(-tiles * 64 // chunk)
        po = torch.full((1, nq, splits, d), float("nan"), device="cuda")
        pml = torch.full((1, nq, splits, 2), float("nan"), device="cuda")
        for tma, cluster in ((False, False), (True, False), (True, True)):
            out = torch.zeros(1, nq * d, dtype=torch.bfloat16, device="cuda")
            ops_attention.decode(q1, nq * d, out, kd, vd, table, ps, i32([0]), i32([last]), slots, 1, nq, nkv, d, window, scale,
                                 chunk, splits, po, pml, tma=tma, cluster=cluster)
            ops_gemm.check_status()
            assert_close(out.view(1, nq, d), want1, f"decode over a long cache, {splits} ranges, tma {tma}, cluster {cluster}", **BF16)


@pytest.mark.parametrize("nq,nkv,d", [(7, 1, 128), (16, 1, 128), (6, 2, 64), (5, 5, 128), (12, 3, 192)])
def test_decode_cluster_merge_for_every_number_of_ranges(nq, nkv, d):
    """The key ranges of a (request, KV head) merged inside a thread-block cluster: every block sends its share of each
    column range to the block that finishes it.  2 to 16 ranges (column ranges that do not divide the head size among
    them), groups of 1 to 16 heads, and beside the long request a short one whose later ranges hold no key at all
    (those blocks send weight zero).  Against the plain formula in float64, and within a last bit of the combine kernel."""
    from tensorline_b200 import ops_attention, ops_gemm
    ps, lens = 16, [1030, 70, 517]                                   # keys each request reads (its own token included)
    B = len(lens)
    ks = [rnd(n, nkv, d, seed=80 + b, dtype=torch.bfloat16) for b, n in enumerate(lens)]
    vs = [rnd(n, nkv, d, seed=90 + b, dtype=torch.bfloat16) for b, n in enumerate(lens)]
    q = rnd(B, nq, d, seed=79, scale=2.0, dtype=torch.bfloat16)
    k_all, v_all = torch.cat(ks), torch.cat(vs)
    num_pages = sum(-(-n // ps) for n in lens) + 9
    # requests laid out one after the other in token order, their pages scattered over the pool
    gen = torch.Generator().manual_seed(11)
    perm = torch.randperm(num_pages, generator=gen).tolist()
    kd = torch.zeros(num_pages + 1, nkv, ps, d, dtype=torch.bfloat16)
    vd = torch.zeros_like(kd)
    rows, used = [], 0
    for b, n in enumerate(lens):
        mine = perm[used:used + -(-n // ps)]
        used += len(mine)
        for t in range(n):
            kd[mine[t // ps], :, t % ps] = ks[b][t]
            vd[mine[t // ps], :, t % ps] = vs[b][t]
        rows.append(mine)
    kd, vd = kd.cuda(), vd.cuda()
    table = table_tensor(rows, 80, num_pages)
    want = torch.cat([_plain_attention_rows(q[b:b + 1].double(), ks[b].double(), vs[b].double(), [lens[b] - 1], None) for b in range(B)])
    qd = q.reshape(B, nq * d).cuda()
    args = (qd, nq * d, None, kd, vd, table, ps, i32(list(range(B))), i32([n - 1 for n in lens]), i32(list(range(B))))
    tiles = -(-max(lens) // 64)
    for ranges in range(2, 17):                              # 9 to 16: clusters beyond the portable size, few requests only
        chunk = -(-tiles // ranges) * 64
        splits = -(-tiles * 64 // chunk)
        if not 2 <= splits <= 16:
            continue
        po = torch.full((B, nq, splits, d), float("nan"), device="cuda")
        pml = torch.full((B, nq, splits, 2), float("nan"), device="cuda")
        outs = []
        for cluster in (True, False):
            out = torch.zeros(B, nq * d, dtype=torch.bfloat16, device="cuda")
            ops_attention.decode(args[0], args[1], out, *args[3:], B, nq, nkv, d, None, d ** -0.5, chunk, splits, po, pml,
                                 tma=True, cluster=cluster)
            ops_gemm.check_status()
            assert_close(out.view(B, nq, d), want, f"{splits} ranges, cluster {cluster}", **BF16)
            outs.append(out)
        # the combine kernel multiplies by a reciprocal where the cluster merge divides: a last bit of bfloat16 at most
        assert_close(outs[0].float(), outs[1].float(), f"{splits} ranges: cluster merge against combine kernel", rtol=2 ** -7, atol=1e-6)


@pytest.mark.parametrize("case", [
    # nq, nkv, d, page, (cached, new tokens) a request, window
    (28, 4, 128, 16, [(1500, 1), (0, 300), (1100, 1), (40, 1)], None),      # singles between and around a portion
    (8, 2, 64, 8, [(70, 2), (1300, 1), (0, 150), (900, 1)], 700),           # a window; the two-token portion stays
    (6, 2, 48, 16, [(1200, 1), (5, 40)], None),                             # a head size without tcgen05 build
    # a portion on a long context that fills little of the GPU: its key tiles are dealt out to two blocks a query-tile pair
    (8, 2, 64, 16, [(3000, 1), (1500, 200), (2900, 1)], None),
    # no single token reads 1.5 times the portion's keys, but their (request, KV head) pairs fill the GPU 1.6 times over
    (40, 8, 128, 16, [(800 + 7 * i, 1) for i in range(30)] + [(900, 260)], None),
])
def test_single_tokens_of_a_mixed_step_take_the_decode_kernel(case, monkeypatch):
    """attend_bf16 on a step of portions beside single decoded tokens: the single tokens with long contexts go
    through the decode kernel (their keys cut into ranges), the portions through a prompt kernel that is told to
    leave them out; every row against the plain formula, and against the same step with everything in the prompt
    kernel."""
    from types import SimpleNamespace
    from tensorline_b200 import ops_attention, ops_gemm
    nq, nkv, d, ps, reqs, window = case
    B = len(reqs)
    max_pages = 256
    num_pages = max(1200, B * (max(c + n for c, n in reqs) // ps + 2))
    kps = torch.zeros(num_pages + 1, nkv, ps, d, dtype=torch.bfloat16)
    vps = torch.zeros_like(kps)
    rows, qs, want, q_start, start_pos = [], [], [], [0], []
    for b, (cached, new) in enumerate(reqs):
        n = cached + new
        k, v = rnd(n, nkv, d, seed=20 + b, dtype=torch.bfloat16), rnd(n, nkv, d, seed=40 + b, dtype=torch.bfloat16)
        q = rnd(new, nq, d, seed=60 + b, scale=2.0, dtype=torch.bfloat16)
        if cached > 600:                            # one far key that must win for the single token
            far = cached - 500
            k[far] *= 0; k[far, :, 0] = 9.0; q[-1] *= 0; q[-1, :, 0] = 9.0
        gen = torch.Generator().manual_seed(100 + b)
        mine = (torch.randperm(num_pages // B, generator=gen)[:-(-n // ps)] * B + b).tolist()
        for i in range(n):
            kps[mine[i // ps], :, i % ps] = k[i]
            vps[mine[i // ps], :, i % ps] = v[i]
        rows.append(mine)
        want.append(_plain_attention_rows(q.double(), k.double(), v.double(), list(range(cached, n)), window))
        qs.append(q)
        q_start.append(q_start[-1] + new)
        start_pos.append(cached)
    T = q_start[-1]
    qkv = torch.zeros(T, (nq + 2 * nkv) * d, dtype=torch.bfloat16)
    qkv[:, :nq * d] = torch.cat(qs).reshape(T, nq * d)
    qkv = qkv.cuda()
    table = table_tensor(rows, max_pages, num_pages)
    kd, vd = kps.cuda(), vps.cuda()

    def run():
        ctx = SimpleNamespace(B=B, T=T, decode_only=False, page_size=ps, q_start=i32(q_start), start_pos=i32(start_pos),
                              slots=i32(list(range(B))), h_q_start=q_start, h_start_pos=start_pos,
                              h_slots=list(range(B)), graph_max_ctx=0, max_ctx=max(c + n for c, n in reqs), scratch={})
        out = torch.zeros(T, nq * d, dtype=torch.bfloat16, device="cuda")
        ops_attention.attend_bf16(qkv, out, ctx, kd, vd, table, nq, nkv, d, window, d ** -0.5)
        ops_gemm.check_status()
        return out, ctx

    out, ctx = run()
    found = ctx.scratch[("single_token_requests", nq // nkv, nkv)]
    assert found is not None and found["set"] == frozenset(b for b, (c, n) in enumerate(reqs) if n == 1)
    assert_close(out.view(T, nq, d), torch.cat(want), "mixed step, single tokens by the decode kernel", **BF16)
    monkeypatch.setattr(ops_attention, "SINGLES_MIN_KEYS", 1 << 30)
    whole, ctx = run()
    assert ctx.scratch[("single_token_requests", nq // nkv, nkv)] is None
    assert_close(whole.view(T, nq, d), torch.cat(want), "mixed step, all in the prompt kernel", **BF16)
    single_rows = [q_start[b] for b, (c, n) in enumerate(reqs) if n == 1]
    other = [r for r in range(T) if r not in single_rows]
    # the portions' rows do not notice, beyond rounding (with the single tokens' tiles another prompt kernel may be chosen,
    # or the key tiles dealt out to several blocks)
    assert_close(out[other].float(), whole[other].float(), "the portion's rows with and without the single tokens beside them", **BF16)


def test_attention_refuses_unsupported_head_size():
    from tensorline_b200 import ops, ops_attention
    with pytest.raises(ops.KernelError):
        ops_attention.attn_lib(24)
    with pytest.raises(ops.KernelError):
        ops_attention.attn_lib(272)


TC_CASES = [  # tokens, N, K, forced (swap, bn, splits) or None for the launcher's plan
    (8, 128, 64, (1, 16, 1)), (8, 200, 1000, (1, 16, 1)), (37, 300, 520, (1, 64, 3)), (1, 3584, 2048, None),
    (16, 4608, 3584, None), (130, 200, 72, (0, 128, 1)), (300, 520, 1000, (0, 256, 1)), (5, 264, 2056, (1, 32, 4)),
    # 64-token tiles: weight and activation tiles in rings of their own, many K tiles a block
    (64, 384, 3000, (1, 64, 1)), (50, 264, 2056, (1, 64, 2)), (130, 200, 1000, (0, 64, 1)), (64, 3584, 18944, None),
]


@pytest.mark.parametrize("case", TC_CASES, ids=[f"T{c[0]}N{c[1]}K{c[2]}" for c in TC_CASES])
@pytest.mark.parametrize("fused", [False, True])
def test_tcgen05_matrix_product(case, fused):
    """The tensor-memory kernel against float64: both operand orders, ragged edges in every dimension,
    K split across blocks with every way of summing the partials (a thread-block cluster, the last block, a
    second kernel), float32 and bfloat16 outputs."""
    from tensorline_b200 import ops_gemm
    T, N, K, forced = case
    x = rnd(T, K, seed=1, dtype=torch.bfloat16).cuda()
    w = rnd(N, K, seed=2, scale=0.1, dtype=torch.bfloat16).cuda()
    want = x.double() @ w.double().T
    kw = dict(zip(("swap", "bn", "splits"), forced)) if forced else {}
    y32 = ops_gemm.gemm_tc(x, w, torch.float32, fused_reduce=fused, **kw)
    y16 = ops_gemm.gemm_tc(x, w, torch.bfloat16, fused_reduce=fused, **kw)
    ops_gemm.check_status()
    if not fused:                                          # K ranges summed by a second kernel instead of a cluster
        assert torch.equal(y32, ops_gemm.gemm_tc(x, w, torch.float32, cluster=False, **kw))
    assert_close(y32, want, "float32 out", rtol=1e-4, atol=1e-4 * float(want.abs().max()))
    assert_close(y16, want, "bfloat16 out", rtol=1e-2, atol=1e-2 * float(want.abs().max()))
    assert int(ops_gemm.status_word(x.device)[1:].abs().sum()) == 0          # arrival counters are back at zero


@pytest.mark.parametrize("rows", [None, [3, 0, 3]])
def test_split_product_summed_inside_the_norm(rows):
    """The pieces of a split-K product handed to the residual add + norm give bit for bit what the
    separate summing pass followed by the norm gives; and the norm part takes a `SplitSum`."""
    from tensorline_b200 import ops, ops_gemm
    from tensorline_b200.parts.linear import SplitSum, resolve
    T, N, K, eps = 5, 264, 2056, 1e-5
    a = rnd(T, K, seed=1, dtype=torch.bfloat16).cuda()
    w = rnd(N, K, seed=2, scale=0.1, dtype=torch.bfloat16).cuda()
    pieces = ops_gemm.gemm_tc(a, w, swap=1, bn=16, splits=4, pieces=True, cluster=False)
    assert pieces.shape == (4, T, N) and pieces.dtype == torch.float32
    whole = ops_gemm.gemm_tc(a, w, swap=1, bn=16, splits=4, cluster=False)
    assert torch.equal(resolve(SplitSum(pieces, torch.bfloat16)), whole)
    # the same four ranges summed inside a thread-block cluster: the same additions in the same order
    assert torch.equal(ops_gemm.gemm_tc(a, w, swap=1, bn=16, splits=4, pieces=True, cluster=True), whole)
    assert torch.equal(ops_gemm.gemm_tc(a, w, torch.float32, swap=1, bn=16, splits=4, cluster=True),
                       ops_gemm.gemm_tc(a, w, torch.float32, swap=1, bn=16, splits=4, cluster=False))
    assert_close(whole, a.double() @ w.double().T, "product", rtol=1e-2, atol=1e-2)
    x = rnd(T, N, seed=3, scale=2.0).cuda()
    nw = (1 + rnd(N, seed=4, scale=0.3)).to(torch.bfloat16).cuda()
    R = T if rows is None else len(rows)
    sel = None if rows is None else i32(rows)
    x1, x2 = x.clone(), x.clone()
    o1 = torch.empty(R, N, dtype=torch.bfloat16, device="cuda")
    o2 = torch.empty_like(o1)
    ops.add_rmsnorm(x1, whole, nw, o1, eps, rows=sel)
    ops.add_rmsnorm(x2, None, nw, o2, eps, rows=sel, pieces=pieces)
    assert torch.equal(o1, o2) and torch.equal(x1, x2)
    if rows is None:
        assert not torch.equal(x1, x)                                          # the sum went into the residual stream
    with pytest.raises(ops.KernelError, match="pieces"):
        ops.add_rmsnorm(x2, whole, nw, o2, eps, rows=sel, pieces=pieces)


def test_tcgen05_matrix_product_refuses_unaligned_k():
    from tensorline_b200 import ops, ops_gemm
    x = torch.zeros(4, 36, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 36, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops_gemm.gemm_tc(x, w)


TC2_CASES = [  # tokens, N, K: ragged edges in every dimension, one tile, many tiles a pair, fewer tiles than pairs
    (256, 256, 64), (300, 384, 200), (65, 136, 72), (513, 640, 1032), (1000, 5000, 520), (2048, 4608, 3584), (96, 20000, 264),
]


@pytest.mark.parametrize("case", TC2_CASES, ids=[f"T{c[0]}N{c[1]}K{c[2]}" for c in TC2_CASES])
def test_two_block_tcgen05_matrix_product(case):
    """The cta_group::2 kernel (pairs of blocks on 256 x 256 tiles, persistent, double-buffered accumulators)
    against float64: float32 and bfloat16 outputs, and with so few pairs that every pair runs many tiles through
    both accumulator buffers."""
    from tensorline_b200 import ops_gemm
    T, N, K = case
    x = rnd(T, K, seed=1, dtype=torch.bfloat16).cuda()
    w = rnd(N, K, seed=2, scale=0.1, dtype=torch.bfloat16).cuda()
    want = x.double() @ w.double().T
    y32 = ops_gemm.gemm_tc2(x, w, torch.float32)
    y16 = ops_gemm.gemm_tc2(x, w, torch.bfloat16)
    few = ops_gemm.gemm_tc2(x, w, torch.float32, max_pairs=3)
    ops_gemm.check_status()
    assert torch.equal(few, y32)                              # a tile's result does not depend on which pair ran it, or when
    assert_close(y32, want, "float32 out", rtol=1e-4, atol=1e-4 * float(want.abs().max()))
    assert_close(y16, want, "bfloat16 out", rtol=1e-2, atol=1e-2 * float(want.abs().max()))
    strided = torch.zeros(T, N + 24, dtype=torch.bfloat16, device="cuda")
    ops_gemm.gemm_tc2(x, w, out=strided[:, 8:8 + N])          # rows further apart than they are wide, unaligned start
    assert torch.equal(strided[:, 8:8 + N], y16) and not bool(strided[:, :8].any()) and not bool(strided[:, 8 + N:].any())


@pytest.mark.parametrize("T,I,K", [(256, 128, 128), (700, 576, 328), (2048, 1216, 904), (70, 64, 64)])
def test_two_block_product_with_the_activation_in_its_epilogue(T, I, K):
    """silu(gate) * up formed in the epilogue from weights whose gate and up rows alternate in blocks of 64 gives
    bit for bit what the product followed by the activation kernel gives (both round gate and up to bfloat16
    first), and agrees with float64."""
    from tensorline_b200 import ops, ops_gemm
    x = rnd(T, K, seed=3, dtype=torch.bfloat16).cuda()
    g = rnd(I, K, seed=4, scale=0.2, dtype=torch.bfloat16)
    u = rnd(I, K, seed=5, scale=0.2, dtype=torch.bfloat16)
    w = torch.stack((g.view(I // 64, 64, K), u.view(I // 64, 64, K)), dim=1).reshape(2 * I, K).contiguous().cuda()
    got = ops_gemm.gemm_tc2(x, w, gated=True)
    ops_gemm.check_status()
    gu = ops_gemm.gemm_tc2(x, w)
    two_pass = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
    ops.silu_mul(gu, two_pass, block=64)
    assert torch.equal(got, two_pass)
    gd, ud = x.double().cpu() @ g.double().T, x.double().cpu() @ u.double().T
    want = gd / (1 + torch.exp(-gd)) * ud
    assert_close(got, want, "gated two-block product", rtol=2e-2, atol=2e-2 * float(want.abs().max()))
    with pytest.raises(ops.KernelError, match="gated"):
        ops_gemm.gemm_tc2(x, w[:64], gated=True)               # 64 rows: a gate block without its up block


@pytest.mark.parametrize("T,N,K,rows", [(8, 3584, 3584, None), (5, 264, 2056, None), (37, 4608, 1024, None), (64, 2560, 520, None),
                                         (16, 1152, 648, None), (32, 4608, 3584, None), (24, 1152, 2056, None), (17, 37888, 3584, None)])
@pytest.mark.parametrize("wdt", [torch.bfloat16, torch.float32])
def test_product_that_normalises_its_operand_on_the_fly(T, N, K, rows, wdt):
    """The few-token product fed with the recipe of a norm's result (residual stream, partial sums of squares, norm
    weight) instead of the result: bit for bit what the product of the same normalised activations gives, when those
    are made with the same rstd (the partial sums added as the kernel adds them: eight lanes, then a butterfly), cast
    before and after the weight as the norm kernel casts."""
    from tensorline_b200 import ops_gemm
    from tensorline_b200.parts.linear import NormedInput
    eps = 1e-5
    R = T if rows is None else 8
    x = rnd(R, K, seed=1, scale=1.5).cuda()
    w = rnd(N, K, seed=2, scale=0.1, dtype=torch.bfloat16).cuda()
    nw = (1 + rnd(K, seed=3, scale=0.2)).to(wdt).cuda()
    parts = 5
    cut = [0, K // 7, K // 3, K // 2, K - 8, K]
    ssq = torch.stack([(x[:, cut[i]:cut[i + 1]] ** 2).sum(-1) for i in range(parts)], dim=1).contiguous()
    sel = None if rows is None else i32(rows)
    v = [ssq[:, p] if p < parts else torch.zeros(R, device="cuda") for p in range(8)]
    total = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]))
    rstd = 1.0 / torch.sqrt(total / K + eps)
    h = ((x * rstd[:, None]).to(torch.bfloat16).float() * nw.float()).to(torch.bfloat16)
    if rows is not None:
        h = h[rows]
    want = ops_gemm.gemm_tc(h.contiguous(), w, torch.float32)
    got = ops_gemm.gemm_tc(NormedInput(x, ssq, nw, eps, sel, torch.bfloat16), w, torch.float32)
    ops_gemm.check_status()
    assert torch.equal(got, want)
    assert_close(got, h.double() @ w.double().T, "normed product", rtol=1e-4, atol=1e-4 * float(want.abs().max()))
    if N % 128 == 0 and ops_gemm.can_gate(T, N, K):          # with the activation in the epilogue as well
        assert torch.equal(ops_gemm.gemm_tc(NormedInput(x, ssq, nw, eps, sel, torch.bfloat16), w, gated=True),
                           ops_gemm.gemm_tc(h.contiguous(), w, gated=True))


@pytest.mark.parametrize("T,N,K", [(8, 3584, 3584), (8, 3584, 18944), (1, 5120, 5120), (37, 1024, 4096), (64, 3584, 2048), (5, 264, 2056)])
def test_product_that_adds_its_result_into_the_residual_stream(T, N, K):
    """The few-token product whose K ranges are summed inside a cluster, adding its result into the float32 residual
    stream itself: the stream becomes bit for bit x + (the product rounded to bfloat16), and the partial sums of squares
    it leaves add up to the squares of the new rows; the norm fed with them agrees with the norm kernel."""
    from tensorline_b200 import ops, ops_gemm
    from tensorline_b200.parts.linear import NormedInput
    if not ops_gemm.can_add_residual(T, N, K):
        pytest.skip("the plan for these sizes has no cluster of 2..8 K ranges")
    a = rnd(T, K, seed=1, dtype=torch.bfloat16).cuda()
    w = rnd(N, K, seed=2, scale=0.05, dtype=torch.bfloat16).cuda()
    x = rnd(T, N, seed=3, scale=2.0).cuda()
    y = ops_gemm.gemm_tc(a, w)                                 # the same ranges, summed in the same order, rounded to bfloat16
    want = x + y.float()
    got = x.clone()
    ssq = ops_gemm.gemm_tc(a, w, residual=got)
    ops_gemm.check_status()
    assert torch.equal(got, want)
    assert ssq.shape == (T, -(-N // 128)) and ssq.dtype == torch.float32
    assert_close(ssq.sum(-1), (want.double() ** 2).sum(-1), "sums of squares", rtol=1e-5, atol=1e-5)
    nw = (1 + rnd(N, seed=4, scale=0.2)).to(torch.bfloat16).cuda()
    h_kernel = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
    ops.add_rmsnorm(want.clone(), None, nw, h_kernel, 1e-6)
    h_recipe = NormedInput(got, ssq, nw, 1e-6, None, torch.bfloat16).materialize()
    assert torch.equal(h_recipe, h_kernel)                    # materialize() is the norm kernel itself
    if N % 8 == 0:
        w2 = rnd(256, N, seed=5, scale=0.05, dtype=torch.bfloat16).cuda()
        fused = ops_gemm.gemm_tc(NormedInput(got, ssq, nw, 1e-6, None, torch.bfloat16), w2, torch.float32)
        plain = ops_gemm.gemm_tc(h_kernel, w2, torch.float32)
        assert_close(fused, plain, "norm folded into the next product", rtol=2e-2, atol=2e-2 * float(plain.abs().max()))


@pytest.mark.parametrize("nq,nkv,d,ps,ctx_lens,window,bias_dt", [
    (28, 4, 128, 16, [300, 0, 63, 64, 1000], None, torch.bfloat16),
    (20, 1, 64, 8, [77, 200, 5, 128], None, torch.float32),          # 20 heads a group: two row tiles a range
    (14, 2, 64, 32, [500, 129, 31, 32], 100, None),                  # a window, no bias
    (7, 1, 128, 64, [15, 16, 2000, 640], None, torch.bfloat16),
])
def test_decode_attention_with_the_rotary_step_folded_in(nq, nkv, d, ps, ctx_lens, window, bias_dt):
    """The TMA decode kernel doing bias, rotation and the page write of the step's own tokens itself gives bit for bit
    what the rotary kernel followed by the decode kernel gives: the same outputs and the same pages, with one key
    range, with ranges merged by the combine kernel and with ranges merged inside clusters."""
    from tensorline_b200 import ops, ops_attention
    B = len(ctx_lens)
    g = torch.Generator().manual_seed(11)
    num_pages, max_pages = 400, 160
    kp = torch.randn(num_pages + 1, nkv, ps, d, generator=g).to(torch.bfloat16).cuda()
    vp = torch.randn(num_pages + 1, nkv, ps, d, generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(num_pages, generator=g).tolist()
    rows, used = [], 0
    for n in ctx_lens:
        need = -(-(n + 1) // ps)
        rows.append(perm[used:used + need]); used += need
    table = table_tensor(rows, max_pages, num_pages)
    qkv = (torch.randn(B, (nq + 2 * nkv) * d, generator=g) * 1.5).to(torch.bfloat16).cuda()
    bias = None if bias_dt is None else (torch.randn((nq + 2 * nkv) * d, generator=g) * 0.5).to(bias_dt).cuda()
    inv_freq = (1e4 ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)).float().cuda()
    pos, slots, q_start = i32(ctx_lens), i32(list(range(B))), i32(list(range(B + 1)))
    span = max(ctx_lens) + 1
    if window:
        span = min(span, window + 63)
    tiles = -(-span // 64)
    for splits_wanted, cluster in ((1, False), (3, False), (3, True), (8, True)):
        splits = min(splits_wanted, tiles)
        chunk = -(-tiles // splits) * 64
        splits = -(-tiles * 64 // chunk)
        if cluster and not 2 <= splits <= 8:
            continue
        po = torch.empty(B, nq, splits, d, device="cuda")
        pml = torch.empty(B, nq, splits, 2, device="cuda")
        # apart: the rotary kernel, then the decode kernel
        q1, k1, v1 = qkv.clone(), kp.clone(), vp.clone()
        ops.rope_kv_write(q1, bias, pos, slots, table, ps, inv_freq, d, nq, nkv, d, k1, v1)
        want = torch.zeros(B, nq * d, dtype=torch.bfloat16, device="cuda")
        ops_attention.decode(q1, q1.shape[1], want, k1, v1, table, ps, q_start, pos, slots, B, nq, nkv, d, window, d ** -0.5,
                             chunk, splits, po, pml, tma=True, cluster=cluster)
        # folded
        k2, v2 = kp.clone(), vp.clone()
        got = torch.zeros_like(want)
        before = ops.kernel_counts.copy()
        ops_attention.decode(qkv, qkv.shape[1], got, k2, v2, table, ps, q_start, pos, slots, B, nq, nkv, d, window, d ** -0.5,
                             chunk, splits, po, pml, tma=True, cluster=cluster,
                             rope={"inv_freq": inv_freq, "bias": bias, "write_kv": True, "unfold": lambda: pytest.fail("turned down")})
        ops.check_device_status()
        assert any(k.startswith("attn_decode_tma+rope") for k in (ops.kernel_counts - before))
        assert torch.equal(k2, k1) and torch.equal(v2, v1), f"pages differ ({splits} ranges, cluster {cluster})"
        assert torch.equal(got, want), f"outputs differ ({splits} ranges, cluster {cluster})"
        assert float(want.float().abs().max()) > 0.05

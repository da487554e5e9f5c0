"""Cases for the checking build of the kernels (-DTL_CHECK=1), run as a program by tests/test_check_build_gpu.py in
a process of its own with TENSORLINE_B200_CHECK=1 (the switch is read when the package is imported).

Each case hands a kernel a block table with an entry outside the bounds the launcher states.  The page tensors the
kernels get are the first `POOL + 1` pages of an allocation that is larger, so the stated bounds are narrower than
the memory: the bad entry would still land inside the allocation even if a check failed to catch it.  The checking
build must record the violation (kernel, value, limit), send the access to the sink page instead, and leave the
pages beyond the stated pool untouched.  Prints one line per case and `ok` at the end.
"""
import sys

import torch


def main() -> int:
    from tensorline_b200 import ops, ops_attention
    from tensorline_b200.csrc.build import CHECK_BUILD
    from tensorline_b200.ops import KernelError
    assert CHECK_BUILD and ops.core().tl_check_build() == 1, "not the checking build"
    dev = torch.device("cuda")
    POOL, REAL, ps, nq, nkv, d = 6, 16, 8, 4, 2, 64
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    real_k = torch.full((REAL, nkv, ps, d), 3.0, dtype=torch.bfloat16, device=dev)
    real_v = torch.full((REAL, nkv, ps, d), -3.0, dtype=torch.bfloat16, device=dev)
    k, v = real_k[:POOL + 1], real_v[:POOL + 1]              # what the kernels are told: pages 0..POOL (POOL is the sink)
    inv_freq = (10000.0 ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)).float().to(dev)
    good = i32([[0, 1, 2, 3], [4, 5, POOL, POOL]])
    bad_page = i32([[0, 9, 2, 3], [4, 5, POOL, POOL]])        # page 9 is outside the stated pool of 7
    T = 3
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=dev).to(torch.bfloat16)

    def expect(what, kernel_word, fn):
        try:
            fn()
            ops.check_device_status()
        except KernelError as e:
            assert "bounds check" in str(e) and kernel_word in str(e), str(e)
            print(f"caught: {what}: {e}")
            return
        raise AssertionError(f"{what}: the checking build reported nothing")

    # a clean call reports nothing
    ops.rope_kv_write(qkv.clone(), None, i32([8, 9, 3]), i32([0, 0, 1]), good, ps, inv_freq, d, nq, nkv, d, k, v)
    ops.check_device_status()
    # rotary + page write: position 9 of slot 0 lives in table entry 1 = page 9
    expect("page number beyond the pool, page write", "rotary",
           lambda: ops.rope_kv_write(qkv.clone(), None, i32([8, 9, 3]), i32([0, 0, 1]), bad_page, ps, inv_freq, d, nq, nkv, d, k, v))
    assert bool((real_k[POOL + 1:] == 3.0).all()) and bool((real_v[POOL + 1:] == -3.0).all()), "a page beyond the pool was written"
    # a request slot beyond the table's rows
    expect("slot beyond the table", "rotary",
           lambda: ops.rope_kv_write(qkv.clone(), None, i32([8, 9, 3]), i32([0, 5, 1]), good, ps, inv_freq, d, nq, nkv, d, k, v))
    # a position beyond the table's width (4 pages of 8)
    expect("position beyond the table's width", "rotary",
           lambda: ops.rope_kv_write(qkv.clone(), None, i32([8, 40, 3]), i32([0, 0, 1]), good, ps, inv_freq, d, nq, nkv, d, k, v))
    assert bool((real_k[POOL + 1:] == 3.0).all())
    # attention kernels reading through the bad entry
    out = torch.zeros(T, nq * d, dtype=torch.bfloat16, device=dev)
    expect("exact-order attention", "exact-order",
           lambda: ops.attn_tokenwise(qkv, qkv.shape[1], out, k, v, bad_page, ps, i32([20, 21, 3]), i32([0, 0, 1]), nq, nkv, d, None, 0.125))
    one = torch.zeros(2, nq * d, dtype=torch.bfloat16, device=dev)
    expect("decode attention", "decode",
           lambda: ops_attention.decode(qkv, qkv.shape[1], one, k, v, bad_page, ps, i32([0, 1, 2]), i32([20, 12]), i32([0, 1]), 2,
                                        nq, nkv, d, None, 0.125, 64, 1, tma=False))
    expect("TMA decode attention", "TMA decode",
           lambda: ops_attention.decode(qkv, qkv.shape[1], one, k, v, bad_page, ps, i32([0, 1, 2]), i32([20, 12]), i32([0, 1]), 2,
                                        nq, nkv, d, None, 0.125, 64, 1, tma=True))
    expect("mma.sync prompt attention", "mma.sync",
           lambda: ops_attention.prefill(qkv, qkv.shape[1], out, k, v, bad_page, ps, i32([0, 2, 3]), i32([18, 3]), i32([0, 1]), [0, 2, 3],
                                         nq, nkv, d, None, 0.125))
    expect("tcgen05 prompt attention", "tcgen05",
           lambda: ops_attention.prefill_tc(qkv, qkv.shape[1], out, k, v, bad_page, ps, i32([0, 2, 3]), i32([18, 3]), i32([0, 1]), [0, 2, 3],
                                            nq, nkv, d, None, 0.125))
    ops.check_device_status()                                # every report was cleared when it was raised
    assert bool((real_k[POOL + 1:] == 3.0).all()) and bool((real_v[POOL + 1:] == -3.0).all())
    print("ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())

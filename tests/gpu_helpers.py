"""Helpers of the GPU tests: stated tolerances, scattered page tables, replay drivers."""
from __future__ import annotations

import torch

# A float32 kernel against the float64 plain implementation, values of order one.
F32 = dict(rtol=2e-5, atol=2e-5)
# A single bfloat16 kernel against float64 on the same (bfloat16-exact) inputs: the output is rounded
# to bfloat16 (2^-9 relative) after float32 accumulation of bfloat16 products.
BF16 = dict(rtol=1.6e-2, atol=1.6e-2)
# Whole model in bfloat16 against the float64 plain model: largest logit error, as a share of the
# largest |logit| of the sequence.  Measured over whole, decoded and cut replays of four sequences per
# model: Tiny A 0.0021, Tiny B 0.0156, B without its window 0.0148, Tiny C 0.0093 (B's weights are drawn
# four times wider than A's, so that attention scores spread over several units).  The bounds are about
# twice the measurement; 0.03 is the bound for a model that has none of its own.
BF16_MODEL_REL = 0.03
BF16_MODEL_REL_OF = {"A": 0.005, "B": 0.03, "B_FULL": 0.03, "C": 0.02}


def scatter_pages(k, v, page_size, num_pages, seed=0, dtype=None, device="cuda"):
    """k, v: [n, nkv, d] (CPU).  Puts them into pages [num_pages + 1, nkv, page, d] in a random page
    order; other pages hold large finite junk, so a read of a wrong page shows.  Returns
    (k_pages, v_pages, table_row list)."""
    n, nkv, d = k.shape
    dtype = dtype or k.dtype
    g = torch.Generator().manual_seed(seed)
    need = -(-n // page_size)
    order = torch.randperm(num_pages, generator=g)[:need].tolist()
    kp = torch.full((num_pages + 1, nkv, page_size, d), 37.0, dtype=dtype)
    vp = torch.full((num_pages + 1, nkv, page_size, d), -53.0, dtype=dtype)
    for i in range(n):
        page, off = order[i // page_size], i % page_size
        kp[page, :, off] = k[i].to(dtype)
        vp[page, :, off] = v[i].to(dtype)
    return kp.to(device), vp.to(device), order


def table_tensor(rows, max_pages, fill, device="cuda"):
    t = torch.full((len(rows), max_pages), fill, dtype=torch.int32)
    for i, r in enumerate(rows):
        t[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
    return t.to(device)


def i32(x, device="cuda"):
    return torch.tensor(x, dtype=torch.int32, device=device)


def assert_close(got, want, what="", **tol):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs()
    bound = tol["atol"] + tol["rtol"] * want.abs()
    if not bool((err <= bound).all()):
        i = int((err - bound).argmax())
        raise AssertionError(f"{what}: max abs err {float(err.max()):.3e}; worst at flat index {i}: "
                             f"got {float(got.flatten()[i]):.6g}, want {float(want.flatten()[i]):.6g}")

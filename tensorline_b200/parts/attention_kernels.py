"""Choice of the attention kernel for a step.

float32: the exact-order kernel for everything.  bfloat16: the tensor-core kernels, one for
steps that hold prompt portions and one (split over the keys) for steps of single decoded
tokens; both read the same pages.  `ctx.force_exact_attention` routes a bfloat16 step through
the exact-order kernel too (tests compare the two).
"""
from __future__ import annotations

import torch

from .. import ops


def attend(mixer, qkv, o, ctx, cache, table, rope=None) -> None:
    nq, nkv, d = mixer.nq, mixer.nkv, mixer.d
    if qkv.dtype == torch.float32 or ctx.force_exact_attention:
        ops.attn_tokenwise(qkv, qkv.shape[1], o, cache.k, cache.v, table, ctx.page_size, ctx.pos, ctx.req_slot,
                           nq, nkv, d, mixer.window, mixer.scale)
        return
    from .. import ops_attention
    ops_attention.attend_bf16(qkv, o, ctx, cache.k, cache.v, table, nq, nkv, d, mixer.window, mixer.scale, rope=rope)

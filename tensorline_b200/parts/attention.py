"""Grouped-query attention over the paged cache: the mixer of this architecture.

Order of work for the T tokens of a step (tensorline/paged.py:248-275):
  qkv = h Wqkv^T                      one product against the stacked q|k|v matrix
  bias, rotary encoding, K/V write    one kernel (tensorline/fused.py:34-51, paged.py:252-253);
                                      every token's k, v are in the pages before any query runs
  attention over the pages            query at position p reads keys lo..p of its own request
                                      (paged.py:237, paged_attn.py:43), scale d^-1/2 (paged.py:119)
  y = o Wo^T                          no bias
The number of heads, of KV heads, the head size, the biases, the window, the position encoding
(with its pairing of dimensions) and an optional RMS norm of every q and k head before the rotation
(`qk_norm_eps`; weights `q_norm.weight`, `k_norm.weight` of the head size) are parameters; the
fused kernel takes all of them as arguments.  A run entry that reads another entry's cache
(`cache.owner` false) computes its own queries and writes no keys or values.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import PagedKV
from .base import POSITION_ENCODINGS, Part, PartSpec, Rotary, Runtime, TensorSpec, register_mixer
from .linear import SplitSum, matmul


@register_mixer("paged_attention")
class PagedAttention(Part):
    graph_capturable = True
    accepts_normed_input = True         # `h` may be a `NormedInput`: the q|k|v product normalises it on the fly

    def __init__(self, rt: Runtime, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position: PartSpec, window: int | None = None, scale: float | None = None,
                 qk_norm_eps: float | None = None):
        super().__init__(rt)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        if head_dim % 16 and not rt.exact:
            raise ValueError(f"head_dim {head_dim}: the bfloat16 attention kernels take multiples of 16")
        self.hidden, self.nq, self.nkv, self.d = hidden, num_heads, num_kv_heads, head_dim
        self.qkv_bias, self.window = qkv_bias, window
        self.scale = head_dim ** -0.5 if scale is None else scale          # tensorline/paged.py:119
        self.position = POSITION_ENCODINGS.build(position, rt, head_dim=head_dim)
        self.qk_norm_eps = qk_norm_eps
        self.w_qkv = self.b_qkv = self.w_o = self.q_norm = self.k_norm = None

    def cache_need(self):
        return PagedKV(self.nkv, self.d, self.window)

    def expected_tensors(self, prefix):
        H, nq, nkv, d = self.hidden, self.nq, self.nkv, self.d
        out = {f"{prefix}.q_proj.weight": TensorSpec((nq * d, H)), f"{prefix}.k_proj.weight": TensorSpec((nkv * d, H)),
               f"{prefix}.v_proj.weight": TensorSpec((nkv * d, H)), f"{prefix}.o_proj.weight": TensorSpec((H, nq * d))}
        if self.qkv_bias:
            out.update({f"{prefix}.q_proj.bias": TensorSpec((nq * d,)), f"{prefix}.k_proj.bias": TensorSpec((nkv * d,)),
                        f"{prefix}.v_proj.bias": TensorSpec((nkv * d,))})
        if self.qk_norm_eps is not None:
            out.update({f"{prefix}.q_norm.weight": TensorSpec((d,), init="ones"),
                        f"{prefix}.k_norm.weight": TensorSpec((d,), init="ones")})
        return out

    def bind(self, weights, prefix):
        w = [weights[f"{prefix}.{n}_proj.weight"] for n in "qkv"]
        self.w_qkv = self._compute_copy(torch.cat(w, dim=0))
        if self.qkv_bias:
            b = [weights[f"{prefix}.{n}_proj.bias"] for n in "qkv"]
            self.b_qkv = torch.cat(b, dim=0).contiguous()
            if self.b_qkv.dtype not in (torch.float32, torch.bfloat16):
                self.b_qkv = self.b_qkv.float()
        self.w_o = self._compute_copy(weights[f"{prefix}.o_proj.weight"])
        if self.qk_norm_eps is not None:
            self.q_norm = weights[f"{prefix}.q_norm.weight"].float().contiguous()
            self.k_norm = weights[f"{prefix}.k_norm.weight"].float().contiguous()

    def forward(self, h, ctx, cache):
        nq, nkv, d = self.nq, self.nkv, self.d
        T = h.shape[0]
        rotary = self.position.rotary()
        if not isinstance(rotary, Rotary):               # a plain (inv_freq, rot) pair means rotate-half pairing
            rotary = Rotary(*rotary)
        inv_freq, rot = rotary.inv_freq, rotary.rot
        plain = rotary.pairing == "half" and self.q_norm is None          # what the kernel's fast path covers
        qkv = matmul(h, self.w_qkv, may_defer=plain and rot == d and d % 16 == 0)
        pieces = None
        if isinstance(qkv, SplitSum):                    # a split-K product: the rotary kernel sums its pieces
            pieces = qkv.pieces
            qkv = torch.empty(qkv.shape, dtype=qkv.dtype, device=h.device)
        table = ctx.tables[cache.group]

        def rotary_kernel():
            ops.rope_kv_write(qkv, self.b_qkv, ctx.pos, ctx.req_slot, table, ctx.page_size, inv_freq, rot,
                              nq, nkv, d, cache.k, cache.v, write_kv=cache.owner, pieces=pieces, pairing=rotary.pairing,
                              q_norm=self.q_norm, k_norm=self.k_norm, norm_eps=self.qk_norm_eps or 0.0)

        # A step of single tokens whose attention kernel can do bias, rotation and the page write of its own tokens
        # (the TMA decode kernel) needs no rotary kernel in front of it.
        fold = None
        if (ctx.decode_only and not ctx.force_exact_attention and qkv.dtype == torch.bfloat16 and pieces is None and plain
                and rot == d and self._folds_rope(ctx)):
            fold = {"inv_freq": inv_freq, "bias": self.b_qkv, "write_kv": cache.owner, "unfold": rotary_kernel}
        else:
            rotary_kernel()
        o = torch.empty((T, nq * d), dtype=qkv.dtype, device=h.device)
        self.attend(qkv, o, ctx, cache, table, rope=fold)
        return matmul(o, self.w_o, may_defer=True, to_residual=True)     # the block's next norm adds it up

    def _folds_rope(self, ctx) -> bool:
        from .. import ops_attention
        return ops_attention.decode_takes_rope(ctx.B, self.d, ctx.page_size)

    def attend(self, qkv, o, ctx, cache, table, rope=None):
        from . import attention_kernels
        attention_kernels.attend(self, qkv, o, ctx, cache, table, rope=rope)

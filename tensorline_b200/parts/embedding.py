"""Token embedding (tensorline/paged.py:240) and the output head (tensorline/paged.py:287)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec, register_embedding, register_head
from .linear import matmul


@register_embedding("token_table")
class Embedding(Part):
    graph_capturable = True

    def __init__(self, rt: Runtime, vocab: int, dim: int):
        super().__init__(rt)
        self.vocab, self.dim = vocab, dim
        self.weight = None

    def expected_tensors(self, prefix):
        return {f"{prefix}.weight": TensorSpec((self.vocab, self.dim))}

    def bind(self, weights, prefix):
        self.weight = self._compute_copy(weights[f"{prefix}.weight"])

    def forward(self, ids):
        """The residual stream starts here, in float32."""
        x = torch.empty((ids.numel(), self.dim), dtype=torch.float32, device=ids.device)
        ops.embed(x, self.weight, ids)
        return x


@register_head("linear")
class LMHead(Part):
    """logits = h W^T in float32, no bias.  Tied: W is the embedding table; a stored
    `lm_head.weight` is then ignored."""
    graph_capturable = True
    accepts_normed_input = True         # `h` may be a `NormedInput`: the product normalises it on the fly

    def __init__(self, rt: Runtime, vocab: int, dim: int, tied: bool):
        super().__init__(rt)
        self.vocab, self.dim, self.tied = vocab, dim, tied
        self.weight = None

    def expected_tensors(self, prefix):
        return {f"{prefix}.weight": TensorSpec((self.vocab, self.dim), optional=self.tied)}

    def bind(self, weights, prefix, embedding: Embedding | None = None):
        if self.tied:
            self.weight = embedding.weight
        else:
            self.weight = self._compute_copy(weights[f"{prefix}.weight"])

    def forward(self, h):
        return matmul(h, self.weight, out_dtype=torch.float32)

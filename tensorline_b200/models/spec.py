"""`ModelSpec`: a model as data, and `Model`, which builds and runs it.

    ModelSpec(vocab, hidden, layers=[LayerSpec...], run=[RunEntry...], final_norm, tied head, ...)

`layers` are the distinct sets of weights; `run` is the order in which they run, one
`RunEntry(layer, cache)` per executed block.  A layer may be named by several entries (shared
weights, each entry with a cache of its own), and an entry may name the cache of an *earlier*
entry in `reads_cache_of` (it then attends to that entry's keys and values and writes none).
The cache manager is told one need per cache-owning entry.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts import BLOCKS, EMBEDDINGS, HEADS, NORMS, POSITION_ENCODINGS, KVCacheView, PartSpec, Runtime


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec                     # params: mixer, feed_forward, norm1, norm2 (PartSpecs)
    prefix: str                         # tensor-name prefix of the layer, e.g. "model.layers.3"


@dataclass(frozen=True)
class RunEntry:
    layer: int                          # index into ModelSpec.layers
    reads_cache_of: int | None = None   # index of an earlier run entry whose cache this one reads


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    layers: tuple
    run: tuple
    final_norm: PartSpec
    tie_word_embeddings: bool
    embedding_prefix: str = "model.embed_tokens"
    final_norm_prefix: str = "model.norm"
    head_prefix: str = "lm_head"
    embedding_position: PartSpec | None = None        # an encoding added to the embedded tokens, if any
    embedding_position_prefix: str = "model.embed_positions"     # where its tensors live, if it has any
    eos_token_id: int | None = None
    max_position_embeddings: int | None = None
    embedding: PartSpec = PartSpec("token_table")     # built with vocab= and dim=; another kind may scale its rows
    head: PartSpec = PartSpec("linear")               # built with vocab=, dim= and tied=; another kind may add a bias or a cap


class Model:
    """The built model: parts on the device, bound to weights; `forward` runs one step."""

    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec, self.rt = spec, rt
        self.embedding = EMBEDDINGS.build(spec.embedding, rt, vocab=spec.vocab_size, dim=spec.hidden_size)
        self.blocks = [BLOCKS.build(l.block, rt) for l in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, rt)
        self.head = HEADS.build(spec.head, rt, vocab=spec.vocab_size, dim=spec.hidden_size, tied=spec.tie_word_embeddings)
        self.embedding_position = (POSITION_ENCODINGS.build(spec.embedding_position, rt)
                                   if spec.embedding_position else None)
        for i, e in enumerate(spec.run):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"run entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            if e.reads_cache_of is not None and not (0 <= e.reads_cache_of < i
                                                     and spec.run[e.reads_cache_of].reads_cache_of is None):
                raise ValueError(f"run entry {i} must read the cache of an earlier entry that owns one")

    # ---- weights
    def expected_tensors(self) -> dict:
        out = dict(self.embedding.expected_tensors(self.spec.embedding_prefix))
        if self.embedding_position is not None:
            out.update(self.embedding_position.expected_tensors(self.spec.embedding_position_prefix))
        for block, layer in zip(self.blocks, self.spec.layers):
            out.update(block.expected_tensors(layer.prefix))
        out.update(self.final_norm.expected_tensors(self.spec.final_norm_prefix))
        out.update(self.head.expected_tensors(self.spec.head_prefix))
        return out

    def bind(self, weights: dict) -> None:
        self.embedding.bind(weights, self.spec.embedding_prefix)
        if self.embedding_position is not None:
            self.embedding_position.bind(weights, self.spec.embedding_position_prefix)
        for block, layer in zip(self.blocks, self.spec.layers):
            block.bind(weights, layer.prefix)
        self.final_norm.bind(weights, self.spec.final_norm_prefix)
        self.head.bind(weights, self.spec.head_prefix, self.embedding)

    # ---- caches
    def cache_needs(self) -> dict:
        """cache id (= index of the owning run entry) -> need."""
        needs = {}
        for i, e in enumerate(self.spec.run):
            if e.reads_cache_of is None:
                need = self.blocks[e.layer].cache_need()
                if need is not None:
                    needs[i] = need
        return needs

    def graph_capturable(self) -> bool:
        """Whether a step of single tokens can be captured in a CUDA graph: every part reads the step from
        device tensors only."""
        parts = [self.embedding, self.final_norm, self.head, *self.blocks]
        if self.embedding_position is not None:
            parts.append(self.embedding_position)
        return all(getattr(p, "graph_capturable", False) for p in parts)

    # ---- one step
    def forward(self, ctx, caches: dict) -> torch.Tensor:
        """Logits [R, V] float32 at the rows `ctx.want_rows`; `caches`: cache id -> view."""
        x = self.embedding.forward(ctx.ids)
        if self.embedding_position is not None:
            self.embedding_position.on_embedding(x, ctx)
        pending = None
        for i, e in enumerate(self.spec.run):
            if e.reads_cache_of is None:
                cache = caches.get(i)
            else:
                owner = caches[e.reads_cache_of]
                cache = KVCacheView(owner.k, owner.v, owner.group, owner=False) if isinstance(owner, KVCacheView) else owner
            pending = self.blocks[e.layer].forward(x, pending, ctx, cache)
        if ctx.want_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        if getattr(self.head, "accepts_normed_input", False) and getattr(self.final_norm, "can_defer", False):
            h = self.final_norm.add_norm(x, pending, rows=ctx.want_rows, defer=True)
        else:
            h = self.final_norm.add_norm(x, pending, rows=ctx.want_rows)
        return self.head.forward(h)

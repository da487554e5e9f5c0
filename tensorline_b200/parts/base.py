"""Interfaces of the parts a layer is put together from, and their registries.

A model is data: a list of layer descriptions, each naming a *block* (the arrangement), a
*mixer* (attention here), a *feed-forward*, its *norms* and the mixer's *position encoding*, every
one a `PartSpec(kind, params)`.  A kind is looked up in the registry of its family and built with
its sizes and constants as keyword parameters; no part knows which model it is in, and a model
may use different kinds in different layers.  Adding a part means: write a class with the
family's interface below and call the family's `register`.

Interfaces (all tensors on the device; T tokens of the step flattened on axis 0):

* Norm            `add_norm(x, pending, rows=None) -> h`: x (float32 residual stream, [T, H]) +=
                  pending (may be None), h = norm(x) in the activation type.  With `rows`
                  (int32 indices) only those rows are produced and x is left alone.
* PositionEncoding `rotary() -> Rotary(inv_freq float32 [rot/2], rot, pairing)` for encodings that
                  rotate q and k inside the mixer (`pairing`: which two dimensions form a pair);
                  `on_embedding(x, ctx)` for encodings added to the embedded tokens.  Either may
                  be a no-op (`rot` = 0).
* Mixer           `cache_need() -> PagedKV | SlotState | None`; `forward(h, ctx, cache) -> y`;
                  `cache` is what the cache manager keeps for this run entry (`KVCacheView`,
                  `StateView` or None), `ctx` the step's `StepContext`.
* FeedForward     `forward(h, ctx) -> y`.
* Block           `forward(x, pending, ctx, cache) -> pending`: runs its norms, mixer and
                  feed-forward; the sum into the residual stream x happens inside the norms.
* Embedding       `forward(ids) -> x`: the float32 residual stream [T, H]; `weight` is the table
                  (a tied head reads it).
* Head            `bind(weights, prefix, embedding)`; `forward(h) -> logits` float32 [R, V].

A part whose `forward` reads the step from device tensors only (never from the host lists of the
`StepContext`, never synchronising) sets `graph_capturable = True`: a model made of such parts
decodes from CUDA graphs.

Every part also declares its tensors, `expected_tensors(prefix) -> {name: TensorSpec}`, and
takes them with `bind(weights, prefix)`.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..weights.loader import TensorSpec


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict = field(default_factory=dict)


@dataclass
class Runtime:
    """What every part needs to know about where it runs."""
    device: torch.device
    act_dtype: torch.dtype              # torch.float32 (true 32-bit engine) or torch.bfloat16
    page_size: int = 16

    @property
    def exact(self) -> bool:
        return self.act_dtype == torch.float32


class Part:
    graph_capturable = False            # True: forward() can be captured in a CUDA graph (see the module text)

    def __init__(self, rt: Runtime):
        self.rt = rt

    def expected_tensors(self, prefix: str) -> dict:
        return {}

    def bind(self, weights: dict, prefix: str) -> None:
        pass

    def _compute_copy(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix as the engine's products read it: the 32-bit engine reads the stored type
        (bfloat16 is widened exactly inside its kernel); the bfloat16 engine needs bfloat16."""
        if self.rt.exact or t.dtype == torch.bfloat16:
            return t.contiguous()
        return t.to(torch.bfloat16).contiguous()


class Registry:
    def __init__(self, family: str):
        self.family = family
        self._kinds: dict = {}

    def register(self, kind: str, factory=None):
        """`register("name", Class)` or as a decorator `@register("name")`."""
        def put(f):
            self._kinds[kind] = f
            return f
        return put(factory) if factory is not None else put

    def build(self, spec: PartSpec, rt: Runtime, **extra):
        if spec.kind not in self._kinds:
            raise KeyError(f"no {self.family} of kind {spec.kind!r}; registered: {sorted(self._kinds)}")
        return self._kinds[spec.kind](rt=rt, **spec.params, **extra)

    def kinds(self):
        return sorted(self._kinds)


@dataclass(frozen=True)
class Rotary:
    """What a rotating position encoding hands to the mixer's fused kernel: angle of pair i at position
    p is p * inv_freq[i]; the first `rot` dimensions of a head are rotated.  `pairing` "half": pair i is
    dimensions (i, i + rot/2) (tensorline/fused.py:47-51); "interleaved": (2i, 2i + 1)."""
    inv_freq: torch.Tensor
    rot: int
    pairing: str = "half"

    def __iter__(self):                 # (inv_freq, rot) = encoding.rotary() still unpacks
        return iter((self.inv_freq, self.rot))

    def __getitem__(self, i):
        return (self.inv_freq, self.rot)[i]


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")

register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register


@dataclass
class KVCacheView:
    """Pages of one run entry: k, v [pages + 1, kv heads, page, d]; `table` is the block table
    of the entry's page group, int32 [slots + 1, max pages], rows indexed by request slot."""
    k: torch.Tensor
    v: torch.Tensor
    group: int
    owner: bool = True                  # False: the entry reads another entry's cache and writes nothing


@dataclass
class StateView:
    """Fixed-size state of one run entry: [slots + 1, *shape], row = request slot."""
    state: torch.Tensor


__all__ = ["PartSpec", "Runtime", "Part", "Registry", "Rotary", "NORMS", "POSITION_ENCODINGS", "MIXERS", "FEED_FORWARDS",
           "BLOCKS", "EMBEDDINGS", "HEADS", "register_norm", "register_position_encoding", "register_mixer",
           "register_feed_forward", "register_block", "register_embedding", "register_head", "KVCacheView",
           "StateView", "TensorSpec"]

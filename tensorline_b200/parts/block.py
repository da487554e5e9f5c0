"""The arrangement of a layer: pre-norm residual block (tensorline/paged.py:245-276).

    h = norm1(x += pending);  a = mixer(h);  h = norm2(x += a);  pending = feed_forward(h)

The sum of a sub-block's output into the residual stream happens inside the next norm
(tensorline/paged.py:247, :275); what the feed-forward returns is handed to the next layer's
first norm (or the model's last) as `pending`.
"""
from __future__ import annotations

from .base import FEED_FORWARDS, MIXERS, NORMS, Part, PartSpec, Runtime, register_block


@register_block("pre_norm")
class PreNormBlock(Part):
    def __init__(self, rt: Runtime, mixer: PartSpec, feed_forward: PartSpec, norm1: PartSpec, norm2: PartSpec,
                 names: dict | None = None):
        super().__init__(rt)
        self.norm1 = NORMS.build(norm1, rt)
        self.mixer = MIXERS.build(mixer, rt)
        self.norm2 = NORMS.build(norm2, rt)
        self.ff = FEED_FORWARDS.build(feed_forward, rt)
        # names of the sub-parts inside the layer's tensor prefix
        self.names = {"norm1": "input_layernorm", "mixer": "self_attn", "norm2": "post_attention_layernorm",
                      "feed_forward": "mlp", **(names or {})}

    def _children(self, prefix):
        n = self.names
        return ((self.norm1, f"{prefix}.{n['norm1']}"), (self.mixer, f"{prefix}.{n['mixer']}"),
                (self.norm2, f"{prefix}.{n['norm2']}"), (self.ff, f"{prefix}.{n['feed_forward']}"))

    def expected_tensors(self, prefix):
        out = {}
        for part, p in self._children(prefix):
            out.update(part.expected_tensors(p))
        return out

    def bind(self, weights, prefix):
        for part, p in self._children(prefix):
            part.bind(weights, p)

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_capturable(self) -> bool:
        return all(part.graph_capturable for part in (self.norm1, self.mixer, self.norm2, self.ff))

    def forward(self, x, pending, ctx, cache):
        # a norm that supports it hands a part that says it can take one (`accepts_normed_input`) the recipe of its
        # result instead of the result (see parts/linear.py)
        h = self._norm(self.norm1, x, pending, self.mixer)
        a = self.mixer.forward(h, ctx, cache)
        h = self._norm(self.norm2, x, a, self.ff)
        return self.ff.forward(h, ctx)

    @staticmethod
    def _norm(norm, x, pending, consumer):
        if getattr(consumer, "accepts_normed_input", False) and getattr(norm, "can_defer", False):
            return norm.add_norm(x, pending, defer=True)
        return norm.add_norm(x, pending)

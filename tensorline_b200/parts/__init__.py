"""Parts of a layer: mixer, feed-forward, norm, position encoding, and their arrangement."""
from .base import (PartSpec, Runtime, Part, Registry, Rotary, NORMS, POSITION_ENCODINGS, MIXERS, FEED_FORWARDS, BLOCKS,
                   EMBEDDINGS, HEADS, register_norm, register_position_encoding, register_mixer,
                   register_feed_forward, register_block, register_embedding, register_head, KVCacheView,
                   StateView, TensorSpec)
from . import norm, rope, mlp, attention, block          # noqa: F401  (registration)
from .embedding import Embedding, LMHead

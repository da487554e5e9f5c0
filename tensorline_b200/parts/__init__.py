"""Parts of a layer: mixer, feed-forward, norm, position encoding, and their arrangement."""
from .base import (PartSpec, Runtime, Part, Registry, NORMS, POSITION_ENCODINGS, MIXERS, FEED_FORWARDS, BLOCKS,
                   register_norm, register_position_encoding, register_mixer, register_feed_forward,
                   register_block, KVCacheView, StateView, TensorSpec)
from . import norm, rope, mlp, attention, block          # noqa: F401  (registration)
from .embedding import Embedding, LMHead

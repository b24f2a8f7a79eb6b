from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS,
                   Arrangement, CacheNeed, Embedding, FeedForward, Head, LayerBinding, Mixer, Norm,
                   Part, PositionEncoding, TensorDecl)
from . import norm, rope, attention, swiglu, block, embedding  # noqa: F401  (register kinds)

from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Arrangement,
                   CacheNeed, LayerBinding, FeedForward, Mixer, Norm, Part, PositionEncoding,
                   TensorDecl)
from . import norm, rope, attention, swiglu, block, embedding  # noqa: F401  (register kinds)

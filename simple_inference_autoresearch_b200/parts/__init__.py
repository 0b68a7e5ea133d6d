"""Parts a decoder layer is put together from, and their registries."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, KVNeed, Mixer,
                   Norm, Part, PartSpec, PositionEncoding, StateNeed, TensorSpec)
from . import attention, block, mlp, norm, rope  # noqa: F401  (register the built-in kinds)

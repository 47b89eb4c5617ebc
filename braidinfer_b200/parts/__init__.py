"""Parts that layers are made of.  Importing the package registers the built-in parts."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                   Block, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Registry)
from .spec import CacheRequest, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
from .runtime import Runtime
from . import attention, block, embedding, feedforward, norm, rope  # noqa: F401  (registration)

"""Parts of a model: embeddings, norms, mixers, feed-forwards, position encodings, heads and the arrangements
of a block, each behind a registry."""
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, CacheNeed, Embedding,
                   FeedForward, Head, Mixer, Norm, ParamDecl, Part, Position, StateNeed, WeightedRows)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from . import attention, block, ends, feed_forward, norm, rope  # noqa: F401  (registers the built-in kinds)

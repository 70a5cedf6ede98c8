"""Parts of a layer: norms, mixers, feed-forwards, position encodings, each behind a registry."""
from .base import (FEED_FORWARDS, MIXERS, NORMS, POSITIONS, CacheNeed, FeedForward, Mixer, Norm, ParamDecl,
                   Part, Position, StateNeed)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from . import attention, feed_forward, norm, rope  # noqa: F401  (registers the built-in kinds)

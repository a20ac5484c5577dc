"""The parts models are put together from.  Importing this package registers the built-in kinds."""

from . import attention, block, embedding, feedforward, norm, position  # noqa: F401
from .base import (  # noqa: F401
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS,
    Block, FeedForward, KVNeed, Mixer, Norm, ParamInfo, Part, PositionEncoding,
    ResidualStream, Runtime, StateNeed, Workspace,
)

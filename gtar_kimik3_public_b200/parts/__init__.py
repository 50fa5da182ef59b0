"""Parts of a model: norms, position encodings, mixers, feed-forwards, blocks, embedding and head.
Importing the package registers the built-in parts."""

from . import attention, block, embedding, mlp, norms, rope  # noqa: F401
from .base import (  # noqa: F401
    Block, FeedForward, KVRequest, Mixer, Norm, Part, PositionEncoding, StateRequest, StepContext, TensorSpec,
    build_part, known_parts, register_part,
)

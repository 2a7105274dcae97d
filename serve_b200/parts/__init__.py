"""Parts a layer is put together from; importing this package registers the built-in ones."""
from .base import (  # noqa: F401
    Block, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, TensorDecl,
    build_part, register_part, registered,
)
from . import norm, rotary, attention, feed_forward, block, embedding  # noqa: F401

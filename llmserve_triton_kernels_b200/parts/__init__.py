"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""

from .base import (  # noqa: F401
    Block,
    CompositeSpec,
    FeedForward,
    Mixer,
    Norm,
    PagedKVSpec,
    PagedRowSpec,
    Part,
    PartSpec,
    PositionEncoding,
    StateSpec,
    TensorSpec,
    build_part,
    register_part,
)
from . import attention, block, feed_forward, latent_attention, norm, parallel, recurrent, rotary, sigmoid_attention, softmax_attention  # noqa: F401,E402

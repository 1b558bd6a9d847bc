"""Parts a layer is put together from: norms, position encodings, mixers, feed-forwards
and block arrangements, each chosen by the ``kind`` of its spec."""
from .base import StepContext
from .registry import (block_class, feed_forward_class, mixer_class, norm_class, position_class,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position, registered)
from . import norms, positions, mixers, feed_forward, blocks  # noqa: F401  (registration)

__all__ = ["StepContext", "block_class", "feed_forward_class", "mixer_class", "norm_class",
           "position_class", "register_block", "register_feed_forward", "register_mixer",
           "register_norm", "register_position", "registered"]

"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards,
block arrangements, and the two ends (embedding, head), each chosen by the ``kind`` of its spec."""
from .base import StepContext
from .registry import (block_class, embedding_class, feed_forward_class, head_class, mixer_class,
                       norm_class, position_class, register_block, register_embedding,
                       register_feed_forward, register_head, register_mixer, register_norm,
                       register_position, registered)
from . import norms, positions, mixers, feed_forward, blocks, ends  # noqa: F401  (registration)

__all__ = ["StepContext", "block_class", "embedding_class", "feed_forward_class", "head_class",
           "mixer_class", "norm_class", "position_class", "register_block", "register_embedding",
           "register_feed_forward", "register_head", "register_mixer", "register_norm",
           "register_position", "registered"]

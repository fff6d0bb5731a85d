from .base import (Arrangement, Embedding, FeedForward, FixedState, Mixer, Norm, PagedKV, Part,
                   PositionEncoding, Precision, StreamShift, build_arrangement, build_embedding,
                   build_feed_forward, build_shift,
                   build_mixer, build_norm, build_position, register_arrangement,
                   register_embedding, register_feed_forward, register_mixer, register_norm,
                   register_position, register_shift, register_side_input)
from . import (attention, block, delta_rule, embedding, latent_attention, linear_attention, mixer_pair, mlp, moe,  # noqa: F401
               norm, outnorm_block, parallel_block, rope, sandwich_block, shortconv, swiglu, token_shift, token_side)  # noqa: F401  (register the parts)

__all__ = [
    "Arrangement", "Embedding", "FeedForward", "FixedState", "Mixer", "Norm", "PagedKV", "Part",
    "PositionEncoding", "Precision", "StreamShift", "build_arrangement", "build_embedding", "build_shift", "build_feed_forward", "build_mixer",
    "build_norm", "build_position", "register_arrangement", "register_feed_forward",
    "register_mixer", "register_norm", "register_position", "register_embedding", "register_shift", "register_side_input",
]

"""Parts of a layer and the registries that build them (see :mod:`.base`)."""
from .base import (Block, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding, Runtime, StateNeed, StreamInput,
                   build_part, known_parts, register_part)
from .stream import ResidualStream
from . import norm, rope, attention, mamba2, gla, latent_attention, diff_attention, feed_forward, experts, block, ends, stream_input  # noqa: F401  (register the built-in kinds)

__all__ = ["Block", "FeedForward", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "StateNeed", "StreamInput",
           "ResidualStream", "build_part", "known_parts", "register_part"]

from . import attention, blocks, feed_forward, io, norms, positions  # noqa: F401  (registers the built-in parts)
from .base import (Block, CacheSpec, FeedForward, Mixer, Norm, Part, PositionEncoding, ResidualStream, StateSpec,
                   TensorSpec, build_part, register_part)
from .model import DecoderModel, Runtime

__all__ = ["Block", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "ResidualStream",
           "StateSpec", "TensorSpec", "build_part", "register_part", "DecoderModel", "Runtime"]

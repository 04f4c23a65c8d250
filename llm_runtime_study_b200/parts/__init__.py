from . import attention, block, differential_attention, experts, gated_attention, gated_recurrence, linear_state, mlp, norm, rope, stream_steps  # registers the built-in kinds
from .base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, FixedState,
    Mixer, Norm, PagedKV, PagedTensors, Part, PositionEncoding, Registry, ResidualStream, Runtime, STREAM_STEPS, StreamStep,
)
from .embedding import OutputHead, TokenEmbedding
from .linear import Projection

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "FeedForward",
    "FixedState", "Mixer", "Norm", "OutputHead", "PagedKV", "PagedTensors", "Part", "STREAM_STEPS", "StreamStep", "PositionEncoding", "Projection",
    "Registry", "ResidualStream", "Runtime", "TokenEmbedding",
]

from . import attention, attention_biased, attention_latent, block, delta, embedding, experts, feed_forward, norm, position, ssm  # noqa: F401  (registers the kinds)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, Embedding,
                   FeedForward, Head, KVNeed, Mixer, Norm, Normed, Part, PartSpec, PositionEncoding, Rotation, Runtime, StateNeed)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block",
           "Embedding", "FeedForward", "Head", "KVNeed", "Mixer", "Norm", "Normed", "Part", "PartSpec", "PositionEncoding",
           "Rotation", "Runtime", "StateNeed"]

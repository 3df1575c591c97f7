from . import attention, attention_biased, attention_latent, block, delta, embedding, experts, feed_forward, norm, position, ssm, stream_entry  # noqa: F401  (registers the kinds)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, STREAM_ENTRIES, Block, Embedding,
                   FeedForward, Head, KVNeed, Mixer, Norm, Normed, Part, PartSpec, PositionEncoding, Rotation, Runtime, StateNeed, StreamEntry)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "STREAM_ENTRIES", "Block",
           "Embedding", "FeedForward", "Head", "KVNeed", "Mixer", "Norm", "Normed", "Part", "PartSpec", "PositionEncoding",
           "Rotation", "Runtime", "StateNeed", "StreamEntry"]

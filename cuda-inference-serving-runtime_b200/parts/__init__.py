"""Parts a model is assembled from: norms, position encodings, mixers, feed-forwards, arrangements."""
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, STREAMS, Embedding, FeedForward,
                   Head, Mixer, Norm, Part, PendingNorm, PositionEncoding, Rotation, TensorNeed, build_part, register)
from . import (attention, block, delta, depth, diff_attention, embedding, experts, feedforward, hyper, latent_attention, lightning, norm, rotary,  # noqa: F401
               windowed_attention)  # noqa: F401  (registers the built-in parts)
from .block import ResidualStream

__all__ = ["ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "STREAMS", "Embedding",
           "FeedForward", "Head", "Mixer", "Norm", "Part", "PendingNorm", "PositionEncoding", "Rotation", "TensorNeed", "build_part",
           "register", "ResidualStream"]

"""The parts a model is assembled from.  Importing the package registers the built-in
kinds; a new kind is added by decorating a class with the registry of its role."""
from . import arrangement, attention, embedding, ffn, norm, rope  # noqa: F401  (registration)
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, REGISTRIES, Arrangement, Delta,
                   Embedding, FeedForward, Head, KVNeed, Mixer, Norm, Part, PositionEncoding, StateNeed, WeightDecl)
from .linear import GatedLinear, Linear
from .spec import LayerSpec, ModelSpec, PartSpec, Run

__all__ = [
    "ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "REGISTRIES",
    "Arrangement", "Delta", "Embedding", "FeedForward", "Head", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding",
    "StateNeed", "WeightDecl", "GatedLinear", "Linear", "LayerSpec", "ModelSpec", "PartSpec", "Run",
]

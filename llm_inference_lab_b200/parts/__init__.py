"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, delta, embedding, latent, mlp, norm, reentry, rope  # noqa: F401  (registration)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, CacheView, Embedding,
                   FeedForward, GroupView, Head, Mixer, Norm, Part, PositionEncoding, StepContext, lookup,
                   register_part)
from .spec import (FixedState, LayerCall, LayerSpec, ModelBlueprint, PagedKV, PagedLatent, PartSpec, Reentry,
                   TensorSpec)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "CacheView",
           "Embedding", "FeedForward", "GroupView", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
           "StepContext", "lookup", "register_part", "FixedState", "LayerCall", "LayerSpec", "ModelBlueprint",
           "PagedKV", "PagedLatent", "PartSpec", "Reentry", "TensorSpec"]

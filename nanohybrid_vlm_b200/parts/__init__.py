from . import (attention, block, delta_rule, embedding, feed_forward, input_filter, latent_attention, linear_recurrence, mlstm, moe, norm,  # noqa: F401
               parallel_mixer, position, sink_attention, state_space)    # (importing registers the built-in parts)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, FILTERS, HEADS, MIXERS, NORMS, POSITIONS, Block, InputFilter, SharedPagesNeed, BuildEnv, CacheView, CompositeNeed,
                   Embedding,
                   FeedForward, FixedStateNeed, Head, Mixer, Norm, PagedKVNeed, Part, Pending, PositionEncoding)
from .spec import LayerRun, LayerSpec, ModelSpec, ParamDecl, PartSpec, PartUse, Source, part

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "FILTERS", "InputFilter", "SharedPagesNeed", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv", "CacheView", "CompositeNeed",
           "Embedding", "FeedForward", "FixedStateNeed", "Head", "Mixer", "Norm", "PagedKVNeed", "Part", "Pending", "PositionEncoding",
           "LayerRun", "LayerSpec", "ModelSpec", "ParamDecl", "PartSpec", "PartUse", "Source", "part"]

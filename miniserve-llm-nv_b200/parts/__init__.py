"""Layer parts and the model assembled from them."""

from . import (attention, block, differential_attention, embedding, experts, feed_forward, latent_attention, linear_recurrence,
               matrix_memory, norm, position, side_by_side, state_space, token_shift)  # noqa: F401  (register the built-in parts)
from .base import (BLOCKS, EMBEDDINGS, ChannelScaled, register_embedding, FEED_FORWARDS, MIXERS, NORMS, PAGED_NEEDS, POSITIONS, FoldedInput, NormFold, PagedKVNeed, PagedLatentNeed, PostNormed,
                   ResidualAdd, ParamSpec, Part, StateNeed,
                   register_block, register_feed_forward, register_mixer, register_norm, register_position)
from .context import PagedKVView, PagedLatentView, StateView, StepContext
from .model import CacheGroup, DecoderModel, RunCache
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec

__all__ = ["BLOCKS", "EMBEDDINGS", "ChannelScaled", "register_embedding", "FEED_FORWARDS", "MIXERS", "NORMS", "PAGED_NEEDS", "POSITIONS", "FoldedInput", "NormFold", "PagedKVNeed",
           "PagedLatentNeed", "PagedLatentView", "PostNormed", "ResidualAdd", "ParamSpec", "Part", "StateNeed", "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "PagedKVView", "StateView", "StepContext", "CacheGroup", "DecoderModel", "RunCache",
           "LayerRun", "LayerSpec", "ModelSpec", "PartSpec"]

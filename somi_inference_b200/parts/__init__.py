"""Parts of a decoder layer, their registries, and the generic decoder built from them."""

from . import (block, conv_attention, embedding, extras, feedforward, latent, mamba2,  # noqa: F401
               matrix_state, mixer, moe, norm, normed_attention, position, side_by_side)  # (register kinds)
from .base import (BranchSum, BuildContext, CacheNeeds, GatedDelta, NormedDelta, PagedKVNeeds,
                   ScaledBranches, StateNeeds, TensorDecl)
from .model import Decoder, declared_tensors
from .registry import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, LAYER_EXTRAS, MIXERS, NORMS,
                       POSITION_ENCODINGS, STREAM_PARTS)

__all__ = ["BranchSum", "STREAM_PARTS", "BuildContext", "CacheNeeds", "GatedDelta", "NormedDelta", "PagedKVNeeds", "ScaledBranches", "StateNeeds", "TensorDecl", "Decoder",
           "declared_tensors", "ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "LAYER_EXTRAS", "MIXERS",
           "NORMS", "POSITION_ENCODINGS"]

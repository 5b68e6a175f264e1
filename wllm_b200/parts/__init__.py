from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, CacheRef, KVNeed, ParamSpec, PartSpec, Partials,
                   Residual, StateNeed, as_branch, spec)
from .plan import LayerRun, ModelPlan
from . import norm, position, attention, feed_forward, embedding, block  # noqa: F401  (register the built-in parts)

__all__ = ["BLOCKS", "EMBEDDINGS", "HEADS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "CacheRef", "KVNeed", "ParamSpec", "PartSpec",
           "Residual", "Partials", "as_branch", "StateNeed", "spec", "LayerRun", "ModelPlan"]

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, CacheRef, KVNeed, MeanOfNormed, NormedBranch,
                   ParamSpec, PartSpec, Partials, Residual, StateNeed, as_branch, branch_pair, spec)
from .plan import LayerRun, ModelPlan
from . import norm, position, attention, linear_attention, latent_attention, feed_forward, embedding, block, hyper_connections, experts  # noqa: F401  (register the built-in parts)

__all__ = ["BLOCKS", "EMBEDDINGS", "HEADS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "CacheRef", "KVNeed", "ParamSpec", "PartSpec",
           "Residual", "Partials", "MeanOfNormed", "NormedBranch", "as_branch", "branch_pair", "StateNeed", "spec", "LayerRun", "ModelPlan"]

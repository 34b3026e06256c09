from . import (attention, block, clamped_glu, embedding, gated_delta, head, latent_attention, lightning, mamba2, masked_attention, moe, norm,
               parallel, pooled_attention, rglru, rope, swiglu, timemix)  # noqa: F401  (registration)
from .base import KVNeed, NeedSet, Part, StateNeed
from .registry import (BuildEnv, register_block, register_embedding, register_ffn, register_head, register_mixer,
                       register_norm, register_positions)

__all__ = ["KVNeed", "NeedSet", "Part", "StateNeed", "BuildEnv", "register_block", "register_embedding", "register_ffn",
           "register_head", "register_mixer", "register_norm", "register_positions"]

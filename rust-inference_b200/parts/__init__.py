"""The parts a model is made of, each behind a registry keyed by ``kind``."""
from .base import (BuildEnv, CacheRequest, FeedForward, Mixer, Norm, Part, Pending, PositionEncoding, StepContext,
                   WeightedSum)
from .registry import (ParamInfo, build_part, part_class, register_block, register_embedding, register_ffn,
                       register_head, register_link, register_mixer, register_norm, register_position, registered)
from . import (attention, ends, gated_delta, gla, latent_attention, link, mlp, mlstm, moe, norm, parallel,  # noqa: F401
               position)                                                      # (registers the built-in parts)
from .block import BlockBase, build_block, norm_before

__all__ = ["BuildEnv", "CacheRequest", "FeedForward", "Mixer", "Norm", "Part", "Pending", "PositionEncoding", "StepContext",
           "ParamInfo", "build_part", "part_class", "register_block", "register_embedding", "register_ffn",
           "register_head", "register_link", "register_mixer", "register_norm", "register_position", "registered",
           "BlockBase", "build_block", "norm_before"]

from .base import (Block, BuildEnv, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding,
                   SubLayer, TensorDecl, build_part, known_parts, part_class, register_part)
from . import attention, block, embedding, gla, latent_attention, mingru, mlp, moe, norm, normed_attention, reentry, rope, sink_attention  # noqa: F401  (registers the built-in parts)

__all__ = ["Block", "BuildEnv", "FeedForward", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding",
           "SubLayer", "TensorDecl", "build_part", "known_parts", "part_class", "register_part"]

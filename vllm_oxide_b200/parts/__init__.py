from .base import (NO_ROTATION, Block, CachePlane, CacheSpec, FeedForward, Mixer, Norm, Part, PartSpec, PositionEncoding,
                   RotationRule, StateSpec, Workspace, build_part, known_parts, register_part)
from . import (attention, block, capped_attention, delta, latent_attention, mlp, moe, norm, parallel, recurrent, rope,  # noqa: F401
               sandwich, streams)  # noqa: F401  (register the built-in parts)
from .linear import linear

__all__ = ["NO_ROTATION", "Block", "CachePlane", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PartSpec",
           "PositionEncoding", "RotationRule", "StateSpec", "Workspace", "build_part", "known_parts", "register_part",
           "linear"]

from .base import (NO_ROTATION, Block, CachePlane, CacheSpec, FeedForward, Mixer, Norm, Part, PartSpec, PositionEncoding,
                   RotationRule, StateSpec, Workspace, build_part, known_parts, register_part)
from . import (attention, block, capped_attention, conv_attention, delta, latent_attention, mlp, moe, norm, parallel,  # noqa: F401
               recurrent, rope, sandwich, side_by_side, streams)  # noqa: F401  (register the built-in parts)
from .linear import linear

__all__ = ["NO_ROTATION", "Block", "CachePlane", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PartSpec",
           "PositionEncoding", "RotationRule", "StateSpec", "Workspace", "build_part", "known_parts", "register_part",
           "linear"]

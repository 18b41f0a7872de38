"""Parts of a layer (mixer, feed-forward, norm, position encoding, arrangement) and the model
that a ModelSpec puts together from them.  Importing this package registers the built-in kinds."""
from .base import (Block, CacheNeed, FeedForward, Mixer, Norm, Part, Position, StateNeed, WeightSpec, build_block,
                   build_part, register_part, registered)
from .spec import Application, LayerSpec, ModelSpec, PartSpec
from . import attention, block, mlp, norm, position  # noqa: F401  (register the built-in kinds)
from .model import DecoderModel

__all__ = ["Application", "Block", "CacheNeed", "DecoderModel", "FeedForward", "LayerSpec", "Mixer", "ModelSpec", "Norm",
           "Part", "PartSpec", "Position", "StateNeed", "WeightSpec", "build_block", "build_part", "register_part",
           "registered"]

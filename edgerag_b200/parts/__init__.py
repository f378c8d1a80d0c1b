"""Parts a decoder is assembled from.  Importing the package registers the built-in kinds."""

from .base import (Block, FeedForward, LayerCall, LayerSpec, Mixer, ModelPlan, Norm, Part, PartSpec,
                   PositionEncoding, WeightSpec, build_part, register_part, registered)
from . import attention, block, embedding, rmsnorm, rope, swiglu  # noqa: F401  (registration)

__all__ = ["Block", "FeedForward", "LayerCall", "LayerSpec", "Mixer", "ModelPlan", "Norm", "Part", "PartSpec",
           "PositionEncoding", "WeightSpec", "build_part", "register_part", "registered"]

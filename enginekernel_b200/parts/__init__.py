"""Parts a layer is put together from; importing this package registers the built-in kinds."""
from . import attention, block, mlp, norm, rope  # noqa: F401
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding, StepContext, Workspace
from .spec import CacheSpec, LayerSpec, ModelSpec, PartSpec, RunSpec, TensorSpec

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "StepContext",
           "Workspace", "CacheSpec", "LayerSpec", "ModelSpec", "PartSpec", "RunSpec", "TensorSpec"]

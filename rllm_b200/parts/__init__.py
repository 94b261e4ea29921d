"""Parts a layer is put together from.  Importing the package registers the
built-in kinds."""
from . import attention, block, mlp, norm, rotary  # noqa: F401  (registration)
from .base import (FeedForward, KVCacheView, Mixer, Norm, Part, PositionEncoding, StateCacheView,
                   StepContext)
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, build_part,
                       register_part)
from .spec import KVPagesNeed, LayerSpec, ModelSpec, PartSpec, Run, StateNeed, TensorSpec

__all__ = ["FeedForward", "KVCacheView", "Mixer", "Norm", "Part", "PositionEncoding", "StateCacheView",
           "StepContext", "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
           "build_part", "register_part", "KVPagesNeed", "LayerSpec", "ModelSpec", "PartSpec", "Run",
           "StateNeed", "TensorSpec"]

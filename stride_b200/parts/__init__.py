from .base import (Block, BuildEnv, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, part_class,
                   register_part)
from .context import ResidualStream, StepContext, Workspace
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorPlan
from . import attention, block, ends, mlp, norm, rope  # register the built-in kinds
from .model import DecoderModel

__all__ = ["Block", "BuildEnv", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "part_class",
           "register_part", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "TensorPlan", "DecoderModel", "ResidualStream", "StepContext", "Workspace"]

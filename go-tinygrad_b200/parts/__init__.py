"""Parts of a model and the plan that arranges them.  Importing this package
registers the parts the library ships with."""
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, default_schedule, plan_weight_specs
from .base import (Block, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding,
                   ResidualStream, Runtime, StepContext, build_part, register_part,
                   registered_parts, unregister_part)
from . import attention, block, embedding, feedforward, norm, position  # noqa: F401  (registration)

__all__ = ["LayerSpec", "ModelPlan", "PartSpec", "ScheduleEntry", "default_schedule",
           "plan_weight_specs", "Block", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part",
           "PositionEncoding", "ResidualStream", "Runtime", "StepContext", "build_part",
           "register_part", "registered_parts", "unregister_part"]

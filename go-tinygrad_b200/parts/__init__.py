"""Parts of a model and the plan that arranges them.  Importing this package
registers the parts the library ships with."""
from .plan import (LayerSpec, ModelPlan, PartSpec, ScheduleEntry, default_schedule, plan_weight_specs,
                   pre_norm_layer)
from .base import (Block, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding,
                   ResidualStream, Runtime, StepContext, build_part, register_part,
                   registered_parts, unregister_part, walk)
from . import attention, block, embedding, feedforward, norm, position  # noqa: F401  (registration)

__all__ = ["LayerSpec", "ModelPlan", "PartSpec", "ScheduleEntry", "default_schedule",
           "plan_weight_specs", "pre_norm_layer", "walk", "Block", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part",
           "PositionEncoding", "ResidualStream", "Runtime", "StepContext", "build_part",
           "register_part", "registered_parts", "unregister_part"]

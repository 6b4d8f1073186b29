from .model import Model, compute_dtype
from .step import StepEntry, StepError, step

__all__ = ["Model", "compute_dtype", "StepEntry", "StepError", "step"]

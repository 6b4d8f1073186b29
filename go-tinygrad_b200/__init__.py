"""go-tinygrad_b200: a small model library with generation of its own for one
GPU (B200, sm_100a) -- configuration, weights, parts, cache, one step function,
a generation loop, sampling and trace replay for the dense Llama decoder.

The package directory carries a hyphen; import it as ``go_tinygrad_b200`` (the
module of that name beside it loads this package).
"""
from . import config, weights, cache, parts, models  # noqa: F401  (models registers architectures)
from .config import ConfigError, LlamaConfig, read_model_config, registered_architectures
from .engine import Model, StepEntry, StepError, step
from .engine.generate import GenerationResult, generate
from .sampling import Sampler
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "LlamaConfig", "read_model_config", "registered_architectures", "Model",
           "StepEntry", "StepError", "step", "WeightError", "write_random_model", "GenerationResult",
           "generate", "Sampler"]

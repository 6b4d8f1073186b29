from .binder import WeightError, WeightSpec, bind, check_specs
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, TensorSource, write_safetensors

__all__ = ["WeightError", "WeightSpec", "bind", "check_specs", "random_tensors", "write_random_model",
           "SafetensorsError", "SafetensorsFile", "TensorSource", "write_safetensors"]

from .loader import (DictSource, SafetensorsSource, TensorSpec, WeightError, WeightSource,
                     bind_tensors, check_tensors)
from .random_weights import RandomSource, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, resolve_shards, write_safetensors

__all__ = ["DictSource", "SafetensorsSource", "TensorSpec", "WeightError", "WeightSource",
           "bind_tensors", "check_tensors", "RandomSource", "write_model_folder",
           "SafetensorsError", "SafetensorsFile", "resolve_shards", "write_safetensors"]

from .loader import (FolderCheckpoint, NamedTensors, TensorSpec, WeightError, check_names,
                     kept_dtype, load_named)
from .random_init import RandomCheckpoint, parse_dtype, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, save_file

__all__ = [
    "FolderCheckpoint", "NamedTensors", "TensorSpec", "WeightError", "check_names", "kept_dtype",
    "load_named", "RandomCheckpoint", "parse_dtype", "write_random_model", "SafetensorsError",
    "SafetensorsFile", "save_file",
]

from .loader import TensorNeed, WeightsError, check_tensors, load_checkpoint
from .random_init import random_tensors, write_model_dir
from .pack import load_packed, pack_model_dir
from .safetensors_io import SafetensorsError, read_file, read_metadata, write_file

__all__ = ["TensorNeed", "WeightsError", "check_tensors", "load_checkpoint",
           "random_tensors", "write_model_dir", "SafetensorsError", "read_file", "read_metadata",
           "write_file", "load_packed", "pack_model_dir"]

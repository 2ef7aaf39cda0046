from .loader import WeightLoadError, convert_tensors, held_dtype, load_tensors, shard_files
from .random_init import random_tensors, write_random_model

__all__ = ["WeightLoadError", "convert_tensors", "held_dtype", "load_tensors", "random_tensors", "shard_files",
           "write_random_model"]

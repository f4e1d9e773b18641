"""Weights: safetensors container, by-name loading with one clear error, random models."""
from .safetensors_io import SafetensorsFile, SafetensorsWriter, SafetensorsError, save_file, find_shards
from .loader import (WeightError, WeightSpec, WeightSource, SafetensorsSource, WeightStore,
                     check_plan, kept_dtype, run_dtype_of)
from .random_init import RandomSource, write_random_model

__all__ = ["SafetensorsFile", "SafetensorsWriter", "SafetensorsError", "save_file", "find_shards",
           "WeightError", "WeightSpec", "WeightSource", "SafetensorsSource", "WeightStore",
           "check_plan", "kept_dtype", "run_dtype_of", "RandomSource", "write_random_model"]

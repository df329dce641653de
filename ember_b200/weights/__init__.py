"""Weights: safetensors container, named loading with collected errors, random-weights mode."""
from .loader import UnexpectedTensorsWarning, WeightError, WeightStore
from .random_init import random_tensors, write_model_dir
from .safetensors_io import SafetensorsDir, SafetensorsError, SafetensorsFile, save_file

__all__ = ["UnexpectedTensorsWarning", "WeightError", "WeightStore", "random_tensors", "write_model_dir", "SafetensorsDir",
           "SafetensorsError", "SafetensorsFile", "save_file"]

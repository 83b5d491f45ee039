"""Weights: safetensors files, binding by name, random model folders."""
from .loader import check, compare, load_checkpoint, target_dtype
from .random_init import random_tensors, write_model_folder
from .safetensors_io import Checkpoint, SafetensorsFile, WeightError, write_safetensors

__all__ = ["Checkpoint", "SafetensorsFile", "WeightError", "check", "compare", "load_checkpoint", "random_tensors",
           "target_dtype", "write_model_folder", "write_safetensors"]

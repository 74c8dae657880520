"""Checkpoints: safetensors files, the by-name loader and the random-weights mode."""

from .decl import TensorDecl
from .safetensors_io import SafetensorsFile, WeightError, write_safetensors
from .loader import Checkpoint, WeightArena, check_tensors, device_dtype, load_checkpoint
from .random_init import random_arena, random_tensor, write_random_model

__all__ = ["TensorDecl", "SafetensorsFile", "WeightError", "write_safetensors", "Checkpoint",
           "WeightArena", "check_tensors", "device_dtype", "load_checkpoint", "random_arena",
           "random_tensor", "write_random_model"]

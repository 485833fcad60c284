"""Checkpoint reading by tensor name, and the random-weights mode."""
from .safetensors_io import CheckpointFormatError, SafetensorsFile, TensorRepository, write_safetensors
from .loader import WeightsError, check_tensors, kept_precision, load_tensors
from .random_init import random_tensors, write_random_model

__all__ = ["CheckpointFormatError", "SafetensorsFile", "TensorRepository", "write_safetensors",
           "WeightsError", "check_tensors", "kept_precision", "load_tensors", "random_tensors",
           "write_random_model"]

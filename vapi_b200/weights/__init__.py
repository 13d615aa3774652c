"""Reading checkpoints and writing random ones."""
from .loader import WeightError, load_tensors, weight_files
from .random import random_tensors, write_random_model

__all__ = ["WeightError", "load_tensors", "weight_files", "random_tensors", "write_random_model"]

"""Weights: the safetensors container, the checked loader, the random-weights mode."""
from .loader import WeightError, check_tensors, load_checked
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, UnreadTensor, read_file, read_folder, read_header, write_file

__all__ = ["SafetensorsError", "UnreadTensor", "WeightError", "check_tensors", "load_checked", "random_tensors", "read_file",
           "read_folder", "read_header", "write_file", "write_random_model"]

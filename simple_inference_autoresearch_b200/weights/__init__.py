"""Weights: safetensors by name (``loader``) and seeded random weights (``random_init``)."""
from .loader import WeightError, check_tensors, load_checkpoint  # noqa: F401
from .random_init import random_tensor, random_tensors, write_model_folder  # noqa: F401

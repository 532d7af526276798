"""Weights: safetensors by tensor name with one clear error, and the random-weights mode."""
from .loader import WeightError, expected_tensors, load_weights, stored_dtype
from .random_init import random_weights, write_random_model

__all__ = ["WeightError", "expected_tensors", "load_weights", "stored_dtype", "random_weights", "write_random_model"]

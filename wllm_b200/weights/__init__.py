from .loader import WeightError, load_weights
from .random_init import fill_random, random_tensors, write_random_model

__all__ = ["WeightError", "load_weights", "fill_random", "random_tensors", "write_random_model"]

from .loader import load_weights, load_state_dict, check_tensors, wanted_tensors, TensorFiles
from .random import random_tensors, write_random_model

__all__ = ["load_weights", "load_state_dict", "check_tensors", "wanted_tensors", "TensorFiles",
           "random_tensors", "write_random_model"]

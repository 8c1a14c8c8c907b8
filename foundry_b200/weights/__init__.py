"""Weights: safetensors by tensor name, the check against a model's list, and
the random-weights mode."""
from .loader import (ExpectedTensor, WeightsMismatch, check_against, load_tensor,
                     stored_to_run_dtype)
from .random_init import random_tensors, write_model_folder
from .safetensors_io import (INDEX_FILE, SINGLE_FILE, WeightFiles, WeightsError, save_file)

__all__ = ["ExpectedTensor", "WeightsMismatch", "check_against", "load_tensor",
           "stored_to_run_dtype", "random_tensors", "write_model_folder", "INDEX_FILE",
           "SINGLE_FILE", "WeightFiles", "WeightsError", "save_file"]

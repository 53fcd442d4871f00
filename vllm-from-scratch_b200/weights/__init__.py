"""Reading checkpoints and making random ones."""

from .loader import (WeightLoadError, check_names, load_weights, load_weights_from_tensors,
                     weight_files)
from .random_init import write_random_model

__all__ = ["WeightLoadError", "check_names", "load_weights", "load_weights_from_tensors",
           "weight_files", "write_random_model"]

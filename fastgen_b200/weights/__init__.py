from .loader import WeightError, checkpoint_files, load_weights
from .random_init import write_random_model

__all__ = ["WeightError", "checkpoint_files", "load_weights", "write_random_model"]

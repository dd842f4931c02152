from .loader import WeightLoadError, checkpoint_names, load_tensors, merge_specs
from .random_init import random_bound_tensors, random_checkpoint_tensors, write_random_model

__all__ = ["WeightLoadError", "checkpoint_names", "load_tensors", "merge_specs",
           "random_bound_tensors", "random_checkpoint_tensors", "write_random_model"]

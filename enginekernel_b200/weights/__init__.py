"""Reading checkpoints by tensor name, and writing seeded random ones."""
from .checkpoint import WeightsError, CheckpointIndex, check_against, read_tensors
from .random_init import random_tensors, write_random_model

__all__ = ["WeightsError", "CheckpointIndex", "check_against", "read_tensors",
           "random_tensors", "write_random_model"]

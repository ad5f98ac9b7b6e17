"""Checkpoint reading and the random-weights writer."""

from turingserve_b200.weights.loader import WeightsError, load_into, load_model, tensor_files
from turingserve_b200.weights.random_init import random_tensors, write_random_model

__all__ = ["WeightsError", "load_into", "load_model", "tensor_files", "random_tensors",
           "write_random_model"]

"""Checkpoints: reading safetensors by tensor name, and writing random ones."""

from gllm_b200.weights.loader import Checkpoint, WeightError, open_checkpoint
from gllm_b200.weights.random_init import write_random_model

__all__ = ["Checkpoint", "WeightError", "open_checkpoint", "write_random_model"]

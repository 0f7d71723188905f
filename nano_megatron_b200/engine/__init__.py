"""Step engine (CUDA-graph captured training step)."""
from .trainer import Trainer

__all__ = ["Trainer"]

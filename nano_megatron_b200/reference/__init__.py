"""Correctness-first single-device GPT used as the numerical oracle."""
from .capture import CaptureLevel, snapshot_grads, snapshot_optimizer, snapshot_params, snapshot_tree
from .config import ReferenceGPTConfig, gpt_preset
from .loss import shifted_cross_entropy
from .model import ReferenceGPT
from .optimizer import AdamW
from .train_step import StepResult, reference_train_loop, reference_train_step, seed_all

__all__ = [
    "AdamW", "CaptureLevel", "ReferenceGPT", "ReferenceGPTConfig", "StepResult", "gpt_preset",
    "reference_train_loop", "reference_train_step", "seed_all", "shifted_cross_entropy",
    "snapshot_grads", "snapshot_optimizer", "snapshot_params", "snapshot_tree",
]

"""Timers, metrics, checkpoints and failure detection."""
from .checkpoint import load_checkpoint, merge_checkpoint, save_checkpoint, shard_tensor, unshard_tensor
from .metrics import JsonlLogger, StepMetrics, gpt_train_flops, measured_peaks, peak_memory_mb, roofline_fraction
from .timers import DeviceTimer, time_steps
from .watchdog import CommTimeout, Heartbeat, StepWatchdog

__all__ = ["CommTimeout", "DeviceTimer", "Heartbeat", "JsonlLogger", "StepMetrics", "StepWatchdog",
           "gpt_train_flops", "load_checkpoint", "measured_peaks", "merge_checkpoint", "peak_memory_mb",
           "roofline_fraction", "save_checkpoint", "shard_tensor", "time_steps", "unshard_tensor"]

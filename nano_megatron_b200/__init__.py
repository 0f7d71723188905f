"""nano_megatron_b200: a Megatron-style training framework written for NVIDIA B200.

Layers (top down): ``schedules`` (1F1B) -> ``models`` (TP/SP/CP GPT, pipeline
stage) -> ``parallel`` (topology, parallel layers, attention backends) ->
``distributed`` (comm backend protocol, DDP, symmetric memory) -> ``ops``
(sm_100a kernels: tcgen05 GEMM and attention, fused norm / CE / embedding /
AdamW) -> ``reference`` (single-device oracle).
"""
__version__ = "0.1.0"

from . import distributed, models, ops, parallel, reference, schedules  # noqa: F401

# The reference project spells the models package ``model``.
model = models

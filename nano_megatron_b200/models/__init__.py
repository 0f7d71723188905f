"""Parallel GPT models built from a full :class:`ReferenceGPT`."""
from .pipeline import PipelineStage, build_pipeline_stage_from_reference
from .tp_gpt import (
    TPGPT,
    TPCausalSelfAttention,
    TPMLP,
    TPTransformerBlock,
    build_tp_gpt_from_reference,
)

__all__ = ["PipelineStage", "TPCausalSelfAttention", "TPGPT", "TPMLP", "TPTransformerBlock",
           "build_pipeline_stage_from_reference", "build_tp_gpt_from_reference"]

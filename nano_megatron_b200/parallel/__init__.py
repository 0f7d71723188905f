"""Topology, tensor/sequence/context-parallel operators and attention backends."""
from .attention_backend import (
    flash_attn_available,
    flash_causal_attention,
    flash_ring_causal_attention,
    resolve_attention_backend,
    unfused_causal_attention,
)
from .config import ParallelConfig
from .context import (
    ParallelContext,
    destroy_parallel,
    get_parallel_context,
    initialize_parallel,
    is_parallel_initialized,
    is_pipeline_first_stage,
    is_pipeline_last_stage,
    pipeline_next_rank,
    pipeline_prev_rank,
)
from .context_parallel import (
    causal_attn_scores_cp,
    gather_from_context_parallel_region,
    local_sequence_range,
    scatter_to_context_parallel_region,
)
from .mappings import (
    ColumnParallelLinear,
    CommunicationBuffer,
    RowParallelLinear,
    blockwise_column_shard,
    column_shard,
    fused_qkv_column_shard,
    gather_from_sequence_parallel_region,
    reduce_scatter_to_sequence_parallel_region,
    register_sequence_parallel_grad_allreduce,
    row_shard,
    scatter_to_sequence_parallel_region,
)
from .rank_generator import RankGenerator, generate_masked_orthogonal_rank_groups
from .vocab_parallel import (
    VocabParallelEmbedding,
    vocab_parallel_cross_entropy,
    vocab_parallel_cross_entropy_from_shifted,
    vocab_range_from_global,
)

__all__ = [
    "ColumnParallelLinear", "CommunicationBuffer", "ParallelConfig", "ParallelContext", "RankGenerator",
    "RowParallelLinear", "VocabParallelEmbedding", "blockwise_column_shard", "causal_attn_scores_cp",
    "column_shard", "destroy_parallel", "flash_attn_available", "flash_causal_attention",
    "flash_ring_causal_attention", "fused_qkv_column_shard", "gather_from_context_parallel_region",
    "gather_from_sequence_parallel_region", "generate_masked_orthogonal_rank_groups", "get_parallel_context",
    "initialize_parallel", "is_parallel_initialized", "is_pipeline_first_stage", "is_pipeline_last_stage",
    "local_sequence_range", "pipeline_next_rank", "pipeline_prev_rank",
    "reduce_scatter_to_sequence_parallel_region", "register_sequence_parallel_grad_allreduce",
    "resolve_attention_backend", "row_shard", "scatter_to_context_parallel_region",
    "scatter_to_sequence_parallel_region", "unfused_causal_attention", "vocab_parallel_cross_entropy",
    "vocab_parallel_cross_entropy_from_shifted", "vocab_range_from_global",
]

"""Parallel layout description (sizes of the TP / PP / CP / DP dimensions).

Same fields, defaults and rejection rules as ``ParallelConfig`` in the
reference (nano_megatron/parallel/config.py:6-65): sequence parallelism cannot
be combined with context parallelism, nor pipeline with context parallelism.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class ParallelConfig:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    context_parallel_size: int = 1
    data_parallel_size: Optional[int] = None
    sequence_parallel: bool = False
    order: str = "tp-cp-dp-pp"

    def _check_positive_sizes(self) -> None:
        for field in ("tensor_parallel_size", "pipeline_parallel_size", "context_parallel_size"):
            if getattr(self, field) < 1:
                raise ValueError(f"{field} must be >= 1")
        if self.data_parallel_size is not None and self.data_parallel_size < 1:
            raise ValueError("data_parallel_size must be >= 1")

    def product_without_dp(self) -> int:
        return self.tensor_parallel_size * self.pipeline_parallel_size * self.context_parallel_size

    def resolved_data_parallel_size(self, world_size: int) -> int:
        self._check_positive_sizes()
        model_ranks = self.product_without_dp()
        if world_size % model_ranks != 0:
            raise ValueError(f"world_size ({world_size}) not divisible by tp*pp*cp ({model_ranks})")
        inferred = world_size // model_ranks
        if self.data_parallel_size is not None and self.data_parallel_size != inferred:
            raise ValueError(
                f"data_parallel_size ({self.data_parallel_size}) inconsistent with "
                f"world_size ({world_size}) / (tp*pp*cp={model_ranks}) = {inferred}"
            )
        return inferred

    def validate(self, world_size: int) -> None:
        self._check_positive_sizes()
        if self.sequence_parallel and self.context_parallel_size > 1:
            raise ValueError("sequence_parallel is not supported with context_parallel_size > 1")
        if self.pipeline_parallel_size > 1 and self.context_parallel_size > 1:
            raise ValueError("pipeline_parallel is not supported with context_parallel_size > 1")
        dp = self.resolved_data_parallel_size(world_size)
        if self.product_without_dp() * dp != world_size:
            raise ValueError(f"world_size ({world_size}) != tp*cp*dp*pp ({self.product_without_dp() * dp})")

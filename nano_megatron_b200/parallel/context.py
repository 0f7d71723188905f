"""Process-wide parallel context: ranks, sizes and process groups.

One process per GPU.  ``initialize_parallel`` brings up ``torch.distributed``
when needed (NCCL on GPUs, Gloo on CPU), validates the layout and creates the
TP / DP / PP / CP / DP x CP groups in the same order on every rank.  Field
names of ``ParallelContext`` and the helper functions match the reference
(nano_megatron/parallel/context.py:16-238) -- tests there build fakes with
``SimpleNamespace`` and ``dataclasses.replace``, so it stays a plain dataclass.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..distributed.backend import CommBackend
from ..distributed.torch_backend import TorchDistBackend
from .config import ParallelConfig
from .rank_generator import RankGenerator


@dataclass
class ParallelContext:
    config: ParallelConfig
    rank: int
    world_size: int
    local_rank: int
    backend: CommBackend
    tensor_parallel_size: int
    tensor_parallel_rank: int
    data_parallel_size: int
    data_parallel_rank: int
    pipeline_parallel_size: int
    pipeline_parallel_rank: int
    context_parallel_size: int
    context_parallel_rank: int
    tensor_parallel_group: Any
    data_parallel_group: Any
    pipeline_parallel_group: Any
    context_parallel_group: Any
    sequence_parallel: bool
    data_context_parallel_group: Any


_CONTEXT: Optional[ParallelContext] = None
_OWNS_PROCESS_GROUP = False

#: Collective timeout given to ``init_process_group``: a rank that never joins
#: ends the others' next collective with an error instead of a hang.
DEFAULT_TIMEOUT_S = float(os.environ.get("NMB_DIST_TIMEOUT_S", "600"))


def _env_int(name: str) -> Optional[int]:
    return int(os.environ[name]) if name in os.environ else None


def _local_rank_for(rank: int) -> int:
    env = _env_int("LOCAL_RANK")
    if env is not None:
        return env
    if torch.cuda.is_available():
        return rank % torch.cuda.device_count()
    return 0


def _my_group(rank: int, rank_lists: list[list[int]]) -> Any:
    """Create every group of one kind (all ranks must make the same calls) and
    return the one that contains ``rank``."""
    mine = None
    for members in rank_lists:
        g = dist.new_group(ranks=members)
        if rank in members:
            mine = g
    if mine is None:
        raise RuntimeError(f"rank {rank} not found in any group of {rank_lists}")
    return mine


def initialize_parallel(
    config: Optional[ParallelConfig] = None,
    *,
    backend: Optional[CommBackend] = None,
    init_method: Optional[str] = None,
    dist_backend: Optional[str] = None,
    rank: Optional[int] = None,
    world_size: Optional[int] = None,
) -> ParallelContext:
    global _CONTEXT, _OWNS_PROCESS_GROUP
    if _CONTEXT is not None:
        raise RuntimeError("parallel context already initialized")
    cfg = config if config is not None else ParallelConfig()

    if dist.is_initialized():
        if world_size is not None and world_size != dist.get_world_size():
            raise RuntimeError(
                f"dist already initialized with world_size={dist.get_world_size()}, got world_size={world_size}")
        if rank is not None and rank != dist.get_rank():
            raise RuntimeError(f"dist already initialized with rank={dist.get_rank()}, got rank={rank}")
    else:
        name = dist_backend or ("nccl" if torch.cuda.is_available() else "gloo")
        want_rank = rank if rank is not None else _env_int("RANK")
        want_world = world_size if world_size is not None else _env_int("WORLD_SIZE")
        if name == "nccl" and torch.cuda.is_available() and (want_rank is not None or "LOCAL_RANK" in os.environ):
            torch.cuda.set_device(_local_rank_for(want_rank or 0))
        kwargs: dict[str, Any] = {"backend": name, "timeout": datetime.timedelta(seconds=DEFAULT_TIMEOUT_S)}
        if init_method is not None:
            kwargs["init_method"] = init_method
        if want_rank is not None:
            kwargs["rank"] = want_rank
        if want_world is not None:
            kwargs["world_size"] = want_world
        dist.init_process_group(**kwargs)
        _OWNS_PROCESS_GROUP = True

    world, me = dist.get_world_size(), dist.get_rank()
    cfg.validate(world)
    dp = cfg.resolved_data_parallel_size(world)
    local_rank = _local_rank_for(me)
    if torch.cuda.is_available() and dist.get_backend() == "nccl":
        torch.cuda.set_device(local_rank)

    gen = RankGenerator(tp=cfg.tensor_parallel_size, dp=dp, pp=cfg.pipeline_parallel_size,
                        cp=cfg.context_parallel_size, order=cfg.order)
    coords = gen.decode(me)
    groups = {tok: _my_group(me, gen.get_ranks(tok)) for tok in ("tp", "dp", "pp", "cp", "dp-cp")}

    _CONTEXT = ParallelContext(
        config=cfg, rank=me, world_size=world, local_rank=local_rank,
        backend=backend if backend is not None else TorchDistBackend(),
        tensor_parallel_size=cfg.tensor_parallel_size, tensor_parallel_rank=coords["tp"],
        data_parallel_size=dp, data_parallel_rank=coords["dp"],
        pipeline_parallel_size=cfg.pipeline_parallel_size, pipeline_parallel_rank=coords["pp"],
        context_parallel_size=cfg.context_parallel_size, context_parallel_rank=coords["cp"],
        tensor_parallel_group=groups["tp"], data_parallel_group=groups["dp"],
        pipeline_parallel_group=groups["pp"], context_parallel_group=groups["cp"],
        sequence_parallel=cfg.sequence_parallel, data_context_parallel_group=groups["dp-cp"],
    )
    return _CONTEXT


def get_parallel_context() -> ParallelContext:
    if _CONTEXT is None:
        raise RuntimeError("parallel context is not initialized")
    return _CONTEXT


def is_parallel_initialized() -> bool:
    return _CONTEXT is not None


def destroy_parallel() -> None:
    global _CONTEXT, _OWNS_PROCESS_GROUP
    _CONTEXT = None
    if dist.is_initialized():
        # peer-mapped buffers go first, while the groups that own them still exist
        from ..distributed import symmetric
        symmetric.close_all()
    if _OWNS_PROCESS_GROUP and dist.is_initialized():
        dist.destroy_process_group()
    _OWNS_PROCESS_GROUP = False


# ----------------------------------------------------- pipeline neighbours --
def _with_pp_rank(ctx: ParallelContext, pp_rank: int) -> int:
    """Global rank with the same tp/cp/dp coordinates on another stage."""
    cfg = getattr(ctx, "config", None)
    order = getattr(cfg, "order", "tp-cp-dp-pp") if cfg is not None else "tp-cp-dp-pp"
    gen = RankGenerator(tp=ctx.tensor_parallel_size, dp=ctx.data_parallel_size, pp=ctx.pipeline_parallel_size,
                        cp=ctx.context_parallel_size, order=order)
    return gen.encode({"tp": ctx.tensor_parallel_rank, "cp": ctx.context_parallel_rank,
                       "dp": ctx.data_parallel_rank, "pp": pp_rank})


def is_pipeline_first_stage(ctx: ParallelContext) -> bool:
    return ctx.pipeline_parallel_rank == 0


def is_pipeline_last_stage(ctx: ParallelContext) -> bool:
    return ctx.pipeline_parallel_rank == ctx.pipeline_parallel_size - 1


def pipeline_prev_rank(ctx: ParallelContext) -> Optional[int]:
    if ctx.pipeline_parallel_size <= 1 or ctx.pipeline_parallel_rank == 0:
        return None
    return _with_pp_rank(ctx, ctx.pipeline_parallel_rank - 1)


def pipeline_next_rank(ctx: ParallelContext) -> Optional[int]:
    if ctx.pipeline_parallel_size <= 1 or is_pipeline_last_stage(ctx):
        return None
    return _with_pp_rank(ctx, ctx.pipeline_parallel_rank + 1)

"""One pipeline stage: embedding on the first stage, an equal slice of the
transformer blocks on every stage, final norm + LM head on the last.

API as in nano_megatron/model/pipeline.py:25-349 (``PipelineStage``,
``build_pipeline_stage_from_reference``, local block names restarting at
``blocks.0``, tied embeddings rejected when ``pp > 1``).  Differences: the stage
is always carved out of a :class:`TPGPT` (so ``tp == 1`` stages run the same
kernels), it is not pinned to fp32 (cast it like any module), and with sequence
parallelism the tensor exchanged between stages is the sequence shard
``[mb, S/t, H]`` -- :meth:`PipelineStage.activation_shape` tells the schedule
what to expect (the reference always receives ``[mb, S, H]``,
nano_megatron/schedules/one_f_one_b.py:111, which is wrong under SP).
"""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch import Tensor, nn
from torch.nn import Parameter

from ..ops import functional as OF
from ..parallel.context import ParallelContext
from ..parallel.vocab_parallel import vocab_parallel_cross_entropy, vocab_range_from_global
from ..reference.config import ReferenceGPTConfig
from ..reference.model import ReferenceGPT
from .tp_gpt import TPGPT, build_tp_gpt_from_reference


def _layer_slice(num_layers: int, pp_rank: int, pp_size: int) -> tuple[int, int]:
    if pp_size < 1:
        raise ValueError(f"pipeline_parallel_size must be >= 1, got {pp_size}")
    if not 0 <= pp_rank < pp_size:
        raise ValueError(f"pipeline_parallel_rank ({pp_rank}) out of range for pp_size={pp_size}")
    if num_layers % pp_size != 0:
        raise ValueError(f"num_layers ({num_layers}) must be divisible by pipeline_parallel_size ({pp_size})")
    per = num_layers // pp_size
    return pp_rank * per, (pp_rank + 1) * per


class PipelineStage(nn.Module):
    def __init__(self, config: ReferenceGPTConfig, *, pp_rank: int, pp_size: int, tok_emb: Optional[nn.Module],
                 pos_emb: Optional[nn.Module], blocks: nn.ModuleList, ln_f_weight: Optional[Parameter],
                 ln_f_bias: Optional[Parameter], lm_head: Optional[nn.Module], tp_rank: int = 0, tp_size: int = 1,
                 tp_group: Any = None, tp_backend: Any = None, sequence_parallel: bool = False) -> None:
        super().__init__()
        self.config = config
        self._pp_rank, self._pp_size = pp_rank, pp_size
        self._tp_rank, self._tp_size = tp_rank, tp_size
        self._tp_group, self._tp_backend = tp_group, tp_backend
        self._sequence_parallel = sequence_parallel
        self.layernorm_eps = config.layernorm_eps
        self.vocab_start_index, self.vocab_end_index = vocab_range_from_global(tp_rank, tp_size, config.vocab_size)
        self.tok_emb = tok_emb
        self.pos_emb = pos_emb
        self.blocks = blocks
        if ln_f_weight is not None:
            self.ln_f_weight = ln_f_weight
        if ln_f_bias is not None:
            self.ln_f_bias = ln_f_bias
        self.lm_head = lm_head
        if self.is_first_stage and self.tok_emb is None:
            raise ValueError("first pipeline stage requires tok_emb")
        if self.is_last_stage and (not hasattr(self, "ln_f_weight") or self.lm_head is None):
            raise ValueError("last pipeline stage requires ln_f_* and lm_head")

    @property
    def is_first_stage(self) -> bool:
        return self._pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self._pp_rank == self._pp_size - 1

    def activation_shape(self, micro_batch: int, seq_len: int) -> tuple[int, int, int]:
        """Shape of the tensor this stage sends / receives for one microbatch."""
        if self._sequence_parallel and self._tp_size > 1:
            return (micro_batch, seq_len // self._tp_size, self.config.hidden_size)
        return (micro_batch, seq_len, self.config.hidden_size)

    def shifted_cross_entropy(self, logits: Tensor, labels: Tensor, ignore_index: int = -100) -> Tensor:
        if not self.is_last_stage:
            raise RuntimeError("shifted_cross_entropy is only valid on the last pipeline stage "
                               f"(pp_rank={self._pp_rank}, pp_size={self._pp_size})")
        if self._tp_size == 1 and not OF.use_native(logits):
            from ..reference.loss import shifted_cross_entropy as plain
            return plain(logits, labels, ignore_index=ignore_index)
        return vocab_parallel_cross_entropy(
            logits, labels, vocab_start_index=self.vocab_start_index, vocab_end_index=self.vocab_end_index,
            group=self._tp_group, backend=self._tp_backend, ignore_index=ignore_index, tp_size=self._tp_size)

    def forward(self, hidden_or_ids: Tensor, *, positions: Optional[Tensor] = None) -> Tensor:
        """First stage: ``input_ids [B, S]``; other stages: activations
        ``[B, S or S/t, H]``.  Last stage returns logits, others activations."""
        if self.is_first_stage:
            ids = hidden_or_ids
            if ids.dim() != 2:
                raise ValueError(f"first stage expects input_ids [B, S], got shape {tuple(ids.shape)}")
            batch, seq_len = ids.shape
            if seq_len > self.config.max_seq_len:
                raise ValueError(f"seq_len ({seq_len}) exceeds max_seq_len ({self.config.max_seq_len})")
            if positions is None:
                positions = torch.arange(seq_len, device=ids.device).unsqueeze(0).expand(batch, -1)
            if self._sequence_parallel and seq_len % self._tp_size != 0:
                raise ValueError(f"seq_len ({seq_len}) must be divisible by tensor_parallel_size "
                                 f"({self._tp_size}) when sequence_parallel is enabled")
            x, _ = TPGPT.embed(self._embed_view(), ids, positions)
        else:
            x = hidden_or_ids
            if x.dim() != 3:
                raise ValueError(f"non-first stage expects hidden [B, S, H], got shape {tuple(x.shape)}")
            batch = x.shape[0]
            seq_len = x.shape[1] * (self._tp_size if self._sequence_parallel else 1)
            if positions is None:
                positions = torch.arange(seq_len, device=x.device).unsqueeze(0).expand(batch, -1)
        for block in self.blocks:
            x = block(x, positions=positions)
        if not self.is_last_stage:
            return x
        if self.config.normalization == "rmsnorm":
            final_ln = OF.rms_norm(x, self.ln_f_weight, self.layernorm_eps)
        else:
            final_ln = OF.layer_norm(x, self.ln_f_weight, self.ln_f_bias, self.layernorm_eps)
        return self.lm_head(final_ln)

    def _embed_view(self):
        """Duck-typed object carrying what ``TPGPT.embed`` reads."""
        from types import SimpleNamespace
        return SimpleNamespace(
            pos_emb=self.pos_emb, tok_emb=self.tok_emb, _cp_size=1, _cp_rank=0,
            _sequence_parallel=self._sequence_parallel, _tp_size=self._tp_size, _tp_rank=self._tp_rank,
            _tp_group=self._tp_group, _tp_backend=self._tp_backend, vocab_start_index=self.vocab_start_index)


def build_pipeline_stage_from_reference(ref: ReferenceGPT, ctx: ParallelContext) -> PipelineStage:
    config = ref.config
    pp_size, pp_rank = ctx.pipeline_parallel_size, ctx.pipeline_parallel_rank
    if config.tie_word_embeddings and pp_size > 1:
        raise ValueError("tie_word_embeddings is not supported when pipeline_parallel_size > 1")
    start, end = _layer_slice(config.num_layers, pp_rank, pp_size)
    full: TPGPT = build_tp_gpt_from_reference(ref, ctx)
    first, last = pp_rank == 0, pp_rank == pp_size - 1
    tok_emb = full.tok_emb if first else None
    pos_emb = full.pos_emb if first else None
    blocks = nn.ModuleList(full.blocks[i] for i in range(start, end))
    lm_head = full.lm_head if last else None
    if last and config.tie_word_embeddings:
        lm_head.weight = tok_emb.weight  # only reachable with pp_size == 1
    stage = PipelineStage(
        config, pp_rank=pp_rank, pp_size=pp_size, tok_emb=tok_emb, pos_emb=pos_emb, blocks=blocks,
        ln_f_weight=full.ln_f_weight if last else None, ln_f_bias=full.ln_f_bias if last else None,
        lm_head=lm_head, tp_rank=ctx.tensor_parallel_rank, tp_size=ctx.tensor_parallel_size,
        tp_group=ctx.tensor_parallel_group, tp_backend=ctx.backend, sequence_parallel=ctx.sequence_parallel)
    del full
    return stage

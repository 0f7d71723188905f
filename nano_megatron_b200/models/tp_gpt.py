"""Tensor / sequence / context-parallel GPT built from a full ``ReferenceGPT``.

Class names, constructor signatures, parameter names and the forward / loss
contract follow nano_megatron/model/tp_gpt.py:52-593, so a state dict maps
one-to-one onto the reference's.  What differs is the execution on a GPU in
bf16: the fused-QKV output is consumed in place by the attention kernel (no
split-heads / merge-heads / repeat-kv copies), bias + GELU and bias + residual
ride in the GEMM epilogues, LayerNorm / embedding / cross entropy are single
kernels, and under context parallelism only the local sequence shard is
embedded (the reference embeds the full sequence on every rank and narrows,
:546-576; the gradients are identical because the narrowed-away rows receive
zero gradient).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor, nn
from torch.nn import Parameter

from ..ops import functional as OF
from ..parallel.attention_backend import (
    flash_causal_attention,
    flash_ring_causal_attention,
    resolve_attention_backend,
    unfused_causal_attention,
)
from ..parallel.context import ParallelContext
from ..parallel.context_parallel import (
    causal_attn_scores_cp,
    gather_from_context_parallel_region,
    local_sequence_range,
    scatter_to_context_parallel_region,
)
from ..parallel.mappings import (
    ColumnParallelLinear,
    RowParallelLinear,
    blockwise_column_shard,
    fused_qkv_column_shard,
    reduce_scatter_to_sequence_parallel_region,
    register_sequence_parallel_grad_allreduce,
    scatter_to_sequence_parallel_region,
)
from ..parallel.vocab_parallel import (
    VocabParallelEmbedding,
    vocab_parallel_cross_entropy,
    vocab_parallel_cross_entropy_from_shifted,
    vocab_range_from_global,
)
from ..reference.config import ReferenceGPTConfig
from ..reference.layers import (
    MLP,
    CausalSelfAttention,
    TransformerBlock,
    apply_rotary_emb,
    precompute_freqs_cis,
    softmax_last,
)
from ..reference.model import ReferenceGPT


def _validate_tp_constraints(config: ReferenceGPTConfig, tp_size: int) -> None:
    if tp_size < 1:
        raise ValueError(f"tensor_parallel_size must be >= 1, got {tp_size}")
    for label, value in (("num_heads", config.num_heads), ("hidden_size", config.hidden_size),
                         ("ffn_hidden_size", config.ffn_hidden_size), ("vocab_size", config.vocab_size)):
        if value is None or value % tp_size != 0:
            raise ValueError(f"{label} ({value}) not divisible by tensor_parallel_size ({tp_size})")
    if config.num_query_groups % tp_size != 0:
        raise ValueError(
            f"num_query_groups ({config.num_query_groups}) not divisible by tensor_parallel_size ({tp_size})")


class TPCausalSelfAttention(nn.Module):
    def __init__(self, ref_attn: CausalSelfAttention, ctx: ParallelContext) -> None:
        super().__init__()
        tp, rank = ctx.tensor_parallel_size, ctx.tensor_parallel_rank
        group, backend, sp = ctx.tensor_parallel_group, ctx.backend, ctx.sequence_parallel
        self.config = ref_attn.config
        self._cp_rank, self._cp_size = ctx.context_parallel_rank, ctx.context_parallel_size
        self._cp_group, self._cp_backend = ctx.context_parallel_group, ctx.backend
        self.num_heads, self.num_kv_heads = ref_attn.num_heads, ref_attn.num_kv_heads
        self.num_heads_per_group = ref_attn.num_heads_per_group
        self.head_dim, self.hidden_size, self.scale = ref_attn.head_dim, ref_attn.hidden_size, ref_attn.scale
        self.local_num_heads = self.num_heads // tp
        self.local_num_kv_heads = self.num_kv_heads // tp
        if self.config.use_fused_qkv:
            w, b = fused_qkv_column_shard(ref_attn.qkv_proj.weight, ref_attn.qkv_proj.bias, rank, tp,
                                          self.hidden_size, self.num_kv_heads * self.head_dim)
            self.qkv_proj = ColumnParallelLinear(w, b, rank, tp, group, backend, weight_is_local=True,
                                                 sequence_parallel=sp)
        else:
            for name in ("q_proj", "k_proj", "v_proj"):
                src = getattr(ref_attn, name)
                setattr(self, name, ColumnParallelLinear(src.weight, src.bias, rank, tp, group, backend,
                                                         sequence_parallel=sp))
        self.out_proj = RowParallelLinear(ref_attn.out_proj.weight, ref_attn.out_proj.bias, rank, tp, group,
                                          backend, sequence_parallel=sp)
        self.rotary_emb = self.config.position_embedding_type == "rope"
        if self.rotary_emb:
            self.freqs = precompute_freqs_cis(self.config.rotary_dim, self.config.max_seq_len,
                                              theta=self.config.rotary_base)
            self._inv_freq_dev: Optional[Tensor] = None

    # -- layout helpers of the generic path ---------------------------------
    def _split_heads(self, x: Tensor, heads: int) -> Tensor:
        b, s, _ = x.shape
        return x.view(b, s, heads, self.head_dim).transpose(1, 2).contiguous()

    def _merge_heads(self, x: Tensor) -> Tensor:
        b, _, s, _ = x.shape
        return x.transpose(1, 2).contiguous().view(b, s, self.local_num_heads * self.head_dim)

    def _repeat_kv(self, x: Tensor, n_rep: int) -> Tensor:
        if n_rep == 1:
            return x
        b, g, s, d = x.shape
        return x[:, :, None].expand(b, g, n_rep, s, d).reshape(b, g * n_rep, s, d)

    def _project(self, x: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        q_size = self.local_num_heads * self.head_dim
        kv_size = self.local_num_kv_heads * self.head_dim
        if self.config.use_fused_qkv:
            return self.qkv_proj(x).split([q_size, kv_size, kv_size], dim=-1)
        return self.q_proj(x), self.k_proj(x), self.v_proj(x)

    def _native_ok(self, x: Tensor) -> bool:
        if not OF.use_native(x) or self.head_dim not in (64, 96, 128):
            return False
        if float(getattr(self.config, "attention_dropout", 0.0)) != 0.0:
            return False
        return resolve_attention_backend(requested=getattr(self.config, "attn_backend", "auto"), dtype=x.dtype,
                                         device=x.device) == "flash"

    def forward(self, x: Tensor, positions: Optional[Tensor] = None, *, residual: Optional[Tensor] = None) -> Tensor:
        if self._native_ok(x):
            return self._forward_native(x, positions, residual)
        q, k, v = self._project(x)
        q = self._split_heads(q, self.local_num_heads)
        k = self._split_heads(k, self.local_num_kv_heads)
        v = self._split_heads(v, self.local_num_kv_heads)
        if self.rotary_emb and positions is not None:
            ang = self.freqs.to(x.device)[positions]
            q, k = apply_rotary_emb(q, ang), apply_rotary_emb(k, ang)
        k = self._repeat_kv(k, self.num_heads_per_group)
        v = self._repeat_kv(v, self.num_heads_per_group)
        backend = resolve_attention_backend(requested=getattr(self.config, "attn_backend", "auto"), dtype=q.dtype,
                                            device=q.device, return_activations=False)
        dropout_p = float(getattr(self.config, "attention_dropout", 0.0))
        if backend == "flash" and self._cp_size > 1:
            context = flash_ring_causal_attention(q, k, v, scale=self.scale, cp_group=self._cp_group,
                                                  cp_rank=self._cp_rank, cp_size=self._cp_size,
                                                  backend=self._cp_backend, dropout_p=dropout_p)
        elif self._cp_size > 1:
            k_full = gather_from_context_parallel_region(k, self._cp_group, self._cp_backend, self._cp_rank,
                                                         self._cp_size, seq_dim=2)
            v_full = gather_from_context_parallel_region(v, self._cp_group, self._cp_backend, self._cp_rank,
                                                         self._cp_size, seq_dim=2)
            scores = causal_attn_scores_cp(q, k_full, scale=self.scale, query_start=self._cp_rank * q.size(2))
            context = torch.matmul(softmax_last(scores), v_full)
        elif backend == "flash":
            context = flash_causal_attention(q, k, v, scale=self.scale, dropout_p=dropout_p)
        else:
            context = unfused_causal_attention(q, k, v, scale=self.scale)
        return self.out_proj(self._merge_heads(context), residual=residual)

    def _rope_spec(self, device: torch.device, positions: Tensor, rope_cols: int):
        """Table of (cos, sin) per position and pair, cached per device, plus the
        flattened positions of this call."""
        from ..ops.gemm import RopeSpec
        table = getattr(self, "_rope_table", None)
        if table is None or table.device != device:
            half = torch.arange(0, self.config.rotary_dim, 2, device=device).float() / self.config.rotary_dim
            inv_freq = 1.0 / (float(self.config.rotary_base) ** half)
            table = RopeSpec.make_table(inv_freq, self.config.max_seq_len)
            self._rope_table = table
        pos = positions.contiguous()
        if pos.dtype != torch.long:
            pos = pos.long()
        return RopeSpec(table, pos, rope_cols)

    def _forward_native(self, x: Tensor, positions: Optional[Tensor], residual: Optional[Tensor]) -> Tensor:
        """bf16 GPU path: packed projection -> in-place views -> tcgen05 attention."""
        from ..ops.attention import flash_attention, flash_attention_packed, split_packed_qkv

        d = self.head_dim
        hq, hkv = self.local_num_heads, self.local_num_kv_heads
        rotate = self.rotary_emb and positions is not None
        if self.config.use_fused_qkv:
            if rotate and self._cp_size == 1 and d % 32 == 0 and self.config.rotary_dim == d:
                # rotary embedding in the projection's epilogue, undone inside the attention
                # backward: no rotation kernel, and the packed layout is kept
                spec = self._rope_spec(x.device, positions, (hq + hkv) * d)
                qkv = self.qkv_proj(x, rope=spec)
                b, s, _ = qkv.shape
                context = flash_attention_packed(qkv.contiguous(), hq, hkv, d, self.scale, rope=spec)
                return self.out_proj(context.view(b, s, hq * d), residual=residual)
            if self._cp_size > 1 and self.qkv_proj.tp_size == 1 and x.dim() == 3 and \
                    (not rotate or (d % 32 == 0 and self.config.rotary_dim == d)):
                from ..distributed import symmetric
                ws = symmetric.workspace_for(self._cp_group)
                if ws is not None and x.shape[1] % 128 == 0:
                    # The projection writes q | k | v into symmetric memory: the peers' attention
                    # kernels read K and V from there in place (no copy into an exchange buffer),
                    # rotary embedding rides in the epilogue and is undone inside the backward.
                    from ..distributed.symm_ops import cp_flash_attention_peer, lease_packed_slot
                    b, s = x.shape[0], x.shape[1]
                    buf, lease = lease_packed_slot(ws, (b, s, (hq + 2 * hkv) * d), x.dtype,
                                                   torch.is_grad_enabled() and x.requires_grad)
                    spec = self._rope_spec(x.device, positions, (hq + hkv) * d) if rotate else None
                    qkv = self.qkv_proj(x, rope=spec, out=buf)
                    q, k, v = split_packed_qkv(qkv, hq, hkv, d)
                    context = cp_flash_attention_peer(q, k, v, self.scale, ws, self._cp_rank, self._cp_size,
                                                      lease, spec)
                    return self.out_proj(context.view(b, s, hq * d), residual=residual)
            qkv = self.qkv_proj(x)
            b, s, _ = qkv.shape
            if self._cp_size == 1 and not rotate and qkv.is_contiguous():
                context = flash_attention_packed(qkv, hq, hkv, d, self.scale)
                return self.out_proj(context.view(b, s, hq * d), residual=residual)
            q, k, v = split_packed_qkv(qkv, hq, hkv, d)
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
            b, s, _ = q.shape
            q, k, v = q.view(b, s, hq, d), k.view(b, s, hkv, d), v.view(b, s, hkv, d)
        if self.rotary_emb and positions is not None:
            if self._inv_freq_dev is None or self._inv_freq_dev.device != x.device:
                half = torch.arange(0, self.config.rotary_dim, 2).float() / self.config.rotary_dim
                self._inv_freq_dev = (1.0 / (float(self.config.rotary_base) ** half)).to(x.device)
            pos = positions.contiguous()
            q = OF.rope_bshd(q, pos, self._inv_freq_dev)
            k = OF.rope_bshd(k, pos, self._inv_freq_dev)
        if self._cp_size > 1:
            from ..parallel.cp_attention import cp_flash_attention
            context = cp_flash_attention(q, k, v, scale=self.scale, cp_group=self._cp_group, cp_rank=self._cp_rank,
                                         cp_size=self._cp_size, backend=self._cp_backend)
        else:
            context = flash_attention(q, k, v, self.scale)
        return self.out_proj(context.view(b, s, hq * d), residual=residual)


class TPMLP(nn.Module):
    def __init__(self, ref_mlp: MLP, ctx: ParallelContext) -> None:
        super().__init__()
        tp, rank = ctx.tensor_parallel_size, ctx.tensor_parallel_rank
        group, backend, sp = ctx.tensor_parallel_group, ctx.backend, ctx.sequence_parallel
        self.config = ref_mlp.config
        if self.config.gated_linear_unit:
            ffn = ref_mlp.fc1.weight.shape[0] // 2
            w, b = blockwise_column_shard(ref_mlp.fc1.weight, ref_mlp.fc1.bias, rank, tp, (ffn, ffn))
            self.fc1 = ColumnParallelLinear(w, b, rank, tp, group, backend, weight_is_local=True, sequence_parallel=sp)
        else:
            self.fc1 = ColumnParallelLinear(ref_mlp.fc1.weight, ref_mlp.fc1.bias, rank, tp, group, backend,
                                            sequence_parallel=sp)
        self.fc2 = RowParallelLinear(ref_mlp.fc2.weight, ref_mlp.fc2.bias, rank, tp, group, backend,
                                     sequence_parallel=sp)

    def forward(self, x: Tensor, *, residual: Optional[Tensor] = None) -> Tensor:
        if self.config.gated_linear_unit:
            if OF.native_linear_ok(x, self.fc1.weight) and OF.swiglu_epilogue_ok(self.fc1.weight):
                # silu(gate) * up in the fc1 epilogue, its backward in the fc2 dgrad epilogue
                pre, act = self.fc1(x, split_act="swiglu")
                return self.fc2(act, residual=residual, act_pre=pre, act="swiglu")
            return self.fc2(OF.swiglu(self.fc1(x)), residual=residual)
        pre, act = self.fc1(x, split_gelu=True)
        return self.fc2(act, residual=residual, gelu_pre=pre)


class TPTransformerBlock(nn.Module):
    def __init__(self, config: ReferenceGPTConfig, ctx: ParallelContext, ref_block: TransformerBlock) -> None:
        super().__init__()
        self.config = config
        self.ln1_weight = Parameter(ref_block.ln1_weight.data.clone())
        self.ln1_bias = Parameter(ref_block.ln1_bias.data.clone())
        self.ln2_weight = Parameter(ref_block.ln2_weight.data.clone())
        self.ln2_bias = Parameter(ref_block.ln2_bias.data.clone())
        self.layernorm_eps = config.layernorm_eps
        self.attn = TPCausalSelfAttention(ref_block.attn, ctx)
        self.mlp = TPMLP(ref_block.mlp, ctx)
        if ctx.sequence_parallel:
            for p in (self.ln1_weight, self.ln1_bias, self.ln2_weight, self.ln2_bias):
                register_sequence_parallel_grad_allreduce(p, ctx.tensor_parallel_group, ctx.backend)

    def _apply_norm(self, x: Tensor, weight: Tensor, bias: Optional[Tensor]) -> Tensor:
        if self.config.normalization == "rmsnorm":
            return OF.rms_norm(x, weight, self.layernorm_eps)
        return OF.layer_norm(x, weight, bias, self.layernorm_eps)

    def forward(self, x: Tensor, positions: Optional[Tensor] = None) -> Tensor:
        rms = self.config.normalization == "rmsnorm"
        h, x = OF.norm_with_residual(x, self.ln1_weight, self.ln1_bias, self.layernorm_eps, rms)
        resid1 = self.attn(h, positions=positions, residual=x)
        h, resid1 = OF.norm_with_residual(resid1, self.ln2_weight, self.ln2_bias, self.layernorm_eps, rms)
        return self.mlp(h, residual=resid1)


class TPGPT(nn.Module):
    def __init__(self, config: ReferenceGPTConfig, ctx: ParallelContext, ref: ReferenceGPT) -> None:
        super().__init__()
        _validate_tp_constraints(config, ctx.tensor_parallel_size)
        self.config = config
        self._tp_group, self._tp_backend = ctx.tensor_parallel_group, ctx.backend
        self._sequence_parallel = ctx.sequence_parallel
        self._tp_rank, self._tp_size = ctx.tensor_parallel_rank, ctx.tensor_parallel_size
        self._cp_rank, self._cp_size = ctx.context_parallel_rank, ctx.context_parallel_size
        self._cp_group, self._cp_backend = ctx.context_parallel_group, ctx.backend
        self.vocab_start_index, self.vocab_end_index = vocab_range_from_global(
            ctx.tensor_parallel_rank, ctx.tensor_parallel_size, config.vocab_size)
        self.tok_emb = VocabParallelEmbedding(config.vocab_size, config.hidden_size, tp_rank=self._tp_rank,
                                              tp_size=self._tp_size, group=self._tp_group, backend=ctx.backend,
                                              weight=ref.tok_emb.weight)
        if config.position_embedding_type == "learned_absolute":
            self.pos_emb = nn.Embedding(config.max_seq_len, config.hidden_size)
            self.pos_emb.weight.data.copy_(ref.pos_emb.weight.data)
        else:
            self.pos_emb = None
        self.blocks = nn.ModuleList(TPTransformerBlock(config, ctx, rb) for rb in ref.blocks)
        self.ln_f_weight = Parameter(ref.ln_f_weight.data.clone())
        self.ln_f_bias = Parameter(ref.ln_f_bias.data.clone())
        self.layernorm_eps = config.layernorm_eps
        if ctx.sequence_parallel:
            sp_params = [self.ln_f_weight, self.ln_f_bias]
            if self.pos_emb is not None:
                sp_params.append(self.pos_emb.weight)  # added on the local sequence shard
            for p in sp_params:
                register_sequence_parallel_grad_allreduce(p, ctx.tensor_parallel_group, ctx.backend)
        self.lm_head = ColumnParallelLinear(ref.lm_head.weight, None, self._tp_rank, self._tp_size, self._tp_group,
                                            ctx.backend, sequence_parallel=ctx.sequence_parallel)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.tok_emb.weight
            # Two kernels (embedding scatter, LM-head wgrad) write this gradient.
            self.tok_emb.weight._nmb_grad_uses = 2
        self.to(dtype=torch.float32)

    # ------------------------------------------------------------------ loss --
    def shifted_cross_entropy(self, logits: Tensor, labels: Tensor, ignore_index: int = -100) -> Tensor:
        """Vocab-parallel shifted CE, mean over non-ignored tokens.

        ``labels`` is the full ``[B, S]`` sequence.  Under CP the logits are the
        local shard ``[B, S/c, V/t]``; each rank scores its own prediction pairs
        and returns ``local_sum * c / global_valid`` so that the DDP mean over
        the DP x CP group recovers the full-sequence mean.
        """
        if self._cp_size == 1:
            return vocab_parallel_cross_entropy(
                logits, labels, vocab_start_index=self.vocab_start_index, vocab_end_index=self.vocab_end_index,
                group=self._tp_group, backend=self._tp_backend, ignore_index=ignore_index, tp_size=self._tp_size)
        if logits.dim() != 3:
            raise ValueError(f"expected logits [B, S_loc, V], got shape {tuple(logits.shape)}")
        if labels.dim() != 2 or labels.shape[0] != logits.shape[0]:
            raise ValueError(f"labels shape {tuple(labels.shape)} incompatible with logits {tuple(logits.shape)}")
        local_seq = logits.shape[1]
        full_seq = local_seq * self._cp_size
        if labels.shape[1] != full_seq:
            raise ValueError(f"labels seq_len ({labels.shape[1]}) must equal full sequence ({full_seq}) under CP; "
                             "CP-local labels are not supported")
        start, end = local_sequence_range(self._cp_rank, self._cp_size, full_seq)
        pred_end = min(end, full_seq - 1)
        if start >= pred_end:
            return logits.sum() * 0.0
        global_valid = (labels[:, 1:] != ignore_index).sum().to(dtype=torch.float32).clamp(min=1.0)
        if OF.use_native(logits):
            # Local logit i pairs with label start+i+1; the global last position
            # gets the ignore label instead of being sliced off.
            local_labels = torch.full((labels.shape[0], local_seq), ignore_index, dtype=labels.dtype,
                                      device=labels.device)
            local_labels[:, : pred_end - start] = labels[:, start + 1: pred_end + 1]
            shift_logits = logits
        else:
            shift_logits = logits[:, : pred_end - start, :].contiguous()
            local_labels = labels[:, start + 1: pred_end + 1].contiguous()
        local_sum = vocab_parallel_cross_entropy_from_shifted(
            shift_logits, local_labels, vocab_start_index=self.vocab_start_index,
            vocab_end_index=self.vocab_end_index, group=self._tp_group, backend=self._tp_backend,
            ignore_index=ignore_index, reduction="sum", tp_size=self._tp_size)
        return local_sum * float(self._cp_size) / global_valid.to(local_sum.dtype)

    # --------------------------------------------------------------- forward --
    def embed(self, input_ids: Tensor, positions: Tensor) -> tuple[Tensor, Tensor]:
        """Token (+ position) embedding of the rows this rank keeps; returns the
        activations and the matching positions."""
        seq_len = input_ids.shape[1]
        pos_w = self.pos_emb.weight if self.pos_emb is not None else None
        if self._cp_size > 1:
            start, end = local_sequence_range(self._cp_rank, self._cp_size, seq_len)
            input_ids, positions = input_ids[:, start:end], positions[:, start:end]
        if self._sequence_parallel and self._tp_size > 1 and OF.use_native(self.tok_emb.weight):
            from ..distributed import symmetric
            ws = symmetric.workspace_for(self._tp_group)
            if ws is not None and self.tok_emb.weight.shape[1] % 8 == 0:
                from ..distributed.symm_ops import sp_embedding
                width = seq_len // self._tp_size
                x = sp_embedding(input_ids, positions if pos_w is not None else None, self.tok_emb.weight, pos_w,
                                 self.vocab_start_index, ws, self)
                return x, positions[:, self._tp_rank * width:(self._tp_rank + 1) * width]
        if self._sequence_parallel and self._tp_size > 1:
            partial = OF.embedding(input_ids, None, self.tok_emb.weight, None, self.vocab_start_index)
            x = reduce_scatter_to_sequence_parallel_region(partial, self._tp_group, self._tp_backend, self._tp_rank,
                                                           self._tp_size)
            width = seq_len // self._tp_size
            positions = positions[:, self._tp_rank * width:(self._tp_rank + 1) * width]
            if pos_w is not None:
                x = x + torch.nn.functional.embedding(positions, pos_w)
            return x, positions
        if self._tp_size > 1 and OF.use_native(self.tok_emb.weight) and self.tok_emb.weight.shape[1] % 8 == 0:
            from ..distributed import symmetric
            ws = symmetric.workspace_for(self._tp_group)
            if ws is not None:
                # the owner of each token's vocabulary id writes the row to every rank (no all-reduce)
                from ..distributed.symm_ops import tp_embedding
                return tp_embedding(input_ids, positions, self.tok_emb.weight, pos_w, self.vocab_start_index,
                                    ws), positions
        x = self.tok_emb(input_ids, positions=positions, pos_weight=pos_w)
        return x, positions

    def forward(self, input_ids: Tensor, positions: Optional[Tensor] = None) -> Tensor:
        batch, seq_len = input_ids.shape
        if seq_len > self.config.max_seq_len:
            raise ValueError(f"seq_len ({seq_len}) exceeds max_seq_len ({self.config.max_seq_len})")
        if positions is None:
            positions = torch.arange(seq_len, device=input_ids.device).unsqueeze(0).expand(batch, -1)
        if self._sequence_parallel and seq_len % self._tp_size != 0:
            raise ValueError(f"seq_len ({seq_len}) must be divisible by tensor_parallel_size ({self._tp_size}) "
                             "when sequence_parallel is enabled")
        if self._cp_size > 1 and seq_len % self._cp_size != 0:
            raise ValueError(f"seq_len ({seq_len}) must be divisible by context_parallel_size ({self._cp_size})")
        if self._cp_size > 1:
            from ..distributed import symmetric
            ws = symmetric.workspace_for(self._cp_group)
            if ws is not None:
                from ..distributed.symm_ops import begin_step
                begin_step(ws)
        x, local_positions = self.embed(input_ids, positions)
        # Under SP attention still sees the full sequence, so the blocks get
        # the full positions; under CP they get the local slice.
        block_positions = positions if self._sequence_parallel else local_positions
        for block in self.blocks:
            x = block(x, positions=block_positions)
        if self.config.normalization == "rmsnorm":
            final_ln = OF.rms_norm(x, self.ln_f_weight, self.layernorm_eps)
        else:
            final_ln = OF.layer_norm(x, self.ln_f_weight, self.ln_f_bias, self.layernorm_eps)
        return self.lm_head(final_ln)


def build_tp_gpt_from_reference(ref: ReferenceGPT, ctx: ParallelContext) -> TPGPT:
    return TPGPT(ref.config, ctx, ref)

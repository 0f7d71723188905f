"""Oracle building blocks: maths helpers and the single-device transformer.

Plain PyTorch, fp32 by construction.  This is the numerical oracle every
parallel path and every CUDA kernel is checked against, and it keeps the
parameter names and the operation order of the reference
(nano_megatron/reference/layers.py:18-365) so that state dicts and
seed-for-seed trajectories are interchangeable.
"""
from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from .config import ReferenceGPTConfig

_INV_SQRT2 = math.sqrt(2.0)


# ------------------------------------------------------------------ helpers --
def layer_norm(x: Tensor, weight: Tensor, bias: Optional[Tensor], eps: float) -> Tensor:
    return F.layer_norm(x, (x.shape[-1],), weight=weight, bias=bias, eps=eps)


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    denom = torch.sqrt(torch.mean(x ** 2, dim=-1, keepdim=True) + eps)
    return x / denom * weight


def gelu_erf(x: Tensor) -> Tensor:
    return 0.5 * x * (1.0 + torch.erf(x / _INV_SQRT2))


def swiglu(x: Tensor) -> Tensor:
    gate, up = x.chunk(2, dim=-1)
    return F.silu(gate) * up


def precompute_freqs_cis(dim: int, max_seq_len: int, theta: float = 10000.0) -> Tensor:
    """Rotary angles ``[max_seq_len, dim/2]`` (fp32)."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2).float() / dim))
    pos = torch.arange(max_seq_len).float()
    return torch.outer(pos, inv)


def apply_rotary_emb(x: Tensor, freqs: Tensor) -> Tensor:
    """Rotate interleaved pairs of ``x[B,h,S,d]`` by ``freqs[B,S,d/2]``."""
    ang = freqs.to(dtype=x.dtype).unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    even, odd = x[..., ::2], x[..., 1::2]
    rot_even = even * c - odd * s
    rot_odd = even * s + odd * c
    return torch.stack([rot_even, rot_odd], dim=-1).flatten(-2)


def causal_attn_scores(q: Tensor, k: Tensor, scale: float) -> Tensor:
    scores = torch.matmul(q, k.transpose(-2, -1)) * scale
    n = scores.size(-1)
    future = torch.triu(torch.ones(n, n, device=scores.device, dtype=torch.bool), diagonal=1)
    return scores.masked_fill(future, torch.finfo(scores.dtype).min)


def softmax_last(x: Tensor) -> Tensor:
    return torch.softmax(x, dim=-1)


# ------------------------------------------------------------------ modules --
class CausalSelfAttention(nn.Module):
    """MHA / GQA with separate or fused ``[Q;K;V]`` projections."""

    def __init__(self, config: ReferenceGPTConfig) -> None:
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_heads
        self.num_query_groups = config.num_query_groups
        self.num_kv_heads = config.num_query_groups
        self.num_heads_per_group = config.num_heads // config.num_query_groups
        self.head_dim = config.hidden_size // config.num_heads
        self.scale = 1.0 / math.sqrt(self.head_dim)
        kv_dim = self.num_kv_heads * self.head_dim
        qkv_bias = bool(config.add_qkv_bias or config.use_bias)
        if config.use_fused_qkv:
            self.qkv_proj = nn.Linear(config.hidden_size, config.hidden_size + 2 * kv_dim, bias=qkv_bias)
        else:
            self.q_proj = nn.Linear(config.hidden_size, config.hidden_size, bias=qkv_bias)
            self.k_proj = nn.Linear(config.hidden_size, kv_dim, bias=qkv_bias)
            self.v_proj = nn.Linear(config.hidden_size, kv_dim, bias=qkv_bias)
        self.out_proj = nn.Linear(config.hidden_size, config.hidden_size, bias=config.use_bias)
        self.rotary_emb = config.position_embedding_type == "rope"
        if self.rotary_emb:
            self.freqs = precompute_freqs_cis(config.rotary_dim, config.max_seq_len, theta=config.rotary_base)
        self.to(dtype=torch.float32)

    def _split_heads(self, x: Tensor, heads: int) -> Tensor:
        b, s, _ = x.shape
        return x.view(b, s, heads, self.head_dim).transpose(1, 2).contiguous()

    def _merge_heads(self, x: Tensor) -> Tensor:
        b, _, s, _ = x.shape
        return x.transpose(1, 2).contiguous().view(b, s, self.hidden_size)

    def _repeat_kv(self, x: Tensor, n_rep: int) -> Tensor:
        if n_rep == 1:
            return x
        b, g, s, d = x.shape
        return x[:, :, None].expand(b, g, n_rep, s, d).reshape(b, g * n_rep, s, d)

    def forward(self, x: Tensor, positions: Optional[Tensor] = None, return_activations: bool = False):
        from ..parallel.attention_backend import (
            flash_causal_attention,
            resolve_attention_backend,
            unfused_causal_attention,
        )

        kv_dim = self.num_kv_heads * self.head_dim
        if self.config.use_fused_qkv:
            q, k, v = self.qkv_proj(x).split([self.hidden_size, kv_dim, kv_dim], dim=-1)
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        q = self._split_heads(q, self.num_heads)
        k = self._split_heads(k, self.num_kv_heads)
        v = self._split_heads(v, self.num_kv_heads)
        if self.rotary_emb and positions is not None:
            ang = self.freqs.to(x.device)[positions]
            q = apply_rotary_emb(q, ang)
            k = apply_rotary_emb(k, ang)
        k = self._repeat_kv(k, self.num_heads_per_group)
        v = self._repeat_kv(v, self.num_heads_per_group)

        backend = resolve_attention_backend(
            requested=self.config.attn_backend, dtype=q.dtype, device=q.device,
            return_activations=return_activations,
        )
        scores = probs = None
        if backend == "flash":
            context = flash_causal_attention(q, k, v, scale=self.scale, dropout_p=self.config.attention_dropout)
        elif return_activations:
            scores = causal_attn_scores(q, k, scale=self.scale)
            probs = softmax_last(scores)
            context = torch.matmul(probs, v)
        else:
            context = unfused_causal_attention(q, k, v, scale=self.scale)
        attn_out = self.out_proj(self._merge_heads(context))
        if not return_activations:
            return attn_out
        return attn_out, {"q": q, "k": k, "v": v, "scores": scores, "probs": probs,
                          "context": context, "attn_out": attn_out}


class MLP(nn.Module):
    def __init__(self, config: ReferenceGPTConfig) -> None:
        super().__init__()
        self.config = config
        width = config.ffn_hidden_size * (2 if config.gated_linear_unit else 1)
        self.fc1 = nn.Linear(config.hidden_size, width, bias=config.use_bias)
        self.fc2 = nn.Linear(config.ffn_hidden_size, config.hidden_size, bias=config.use_bias)
        self.to(dtype=torch.float32)

    def forward(self, x: Tensor, return_activations: bool = False):
        h = self.fc1(x)
        h = swiglu(h) if self.config.gated_linear_unit else gelu_erf(h)
        out = self.fc2(h)
        if not return_activations:
            return out
        return out, {"fc1_gelu": h, "mlp_out": out}


class TransformerBlock(nn.Module):
    """Pre-norm block; the norm parameters are bare ``nn.Parameter`` s."""

    def __init__(self, config: ReferenceGPTConfig) -> None:
        super().__init__()
        self.config = config
        h = config.hidden_size
        self.ln1_weight = nn.Parameter(torch.ones(h))
        self.ln1_bias = nn.Parameter(torch.zeros(h))
        self.ln2_weight = nn.Parameter(torch.ones(h))
        self.ln2_bias = nn.Parameter(torch.zeros(h))
        self.layernorm_eps = config.layernorm_eps
        self.attn = CausalSelfAttention(config)
        self.mlp = MLP(config)
        self.to(dtype=torch.float32)

    def _apply_norm(self, x: Tensor, weight: Tensor, bias: Optional[Tensor]) -> Tensor:
        if self.config.normalization == "rmsnorm":
            return rms_norm(x, weight, self.layernorm_eps)
        return layer_norm(x, weight, bias, self.layernorm_eps)

    def forward(self, x: Tensor, positions: Optional[Tensor] = None, return_activations: bool = False):
        ln1_out = self._apply_norm(x, self.ln1_weight, self.ln1_bias)
        attn_acts = mlp_acts = None
        if return_activations:
            attn_out, attn_acts = self.attn(ln1_out, positions=positions, return_activations=True)
        else:
            attn_out = self.attn(ln1_out, positions=positions)
        resid1 = x + attn_out
        ln2_out = self._apply_norm(resid1, self.ln2_weight, self.ln2_bias)
        if return_activations:
            mlp_out, mlp_acts = self.mlp(ln2_out, return_activations=True)
        else:
            mlp_out = self.mlp(ln2_out)
        resid2 = resid1 + mlp_out
        if not return_activations:
            return resid2
        acts: dict[str, Any] = {"ln1_out": ln1_out, "attn_out": attn_out, "resid1": resid1,
                                "ln2_out": ln2_out, "mlp_out": mlp_out, "resid2": resid2}
        if attn_acts is not None:
            acts["attn"] = attn_acts
        if mlp_acts is not None:
            acts["mlp"] = mlp_acts
        return resid2, acts

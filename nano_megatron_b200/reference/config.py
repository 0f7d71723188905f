"""Model hyper-parameters shared by the oracle GPT and the parallel models.

Field names, defaults and validation follow ``ReferenceGPTConfig`` of the
reference project (nano_megatron/reference/config.py:7-55) so that a config
object written for one can be passed to the other.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional

import torch


@dataclass
class ReferenceGPTConfig:
    vocab_size: int = 51200
    max_seq_len: int = 1024
    hidden_size: int = 512
    num_layers: int = 12
    num_heads: int = 8
    ffn_hidden_size: Optional[int] = None
    layernorm_eps: float = 1e-5
    use_bias: bool = False
    tie_word_embeddings: bool = False
    dtype: torch.dtype = torch.float32

    position_embedding_type: Literal["learned_absolute", "rope"] = "rope"
    rotary_dim: Optional[int] = None
    rotary_base: int = 10000
    activation_func: Literal["gelu", "swiglu"] = "swiglu"  # informational; see gated_linear_unit
    use_fused_qkv: bool = False
    num_query_groups: Optional[int] = None
    add_qkv_bias: bool = False
    gated_linear_unit: bool = True
    normalization: Literal["layernorm", "rmsnorm"] = "layernorm"
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    attn_backend: Literal["auto", "flash", "unfused"] = "auto"

    def __post_init__(self) -> None:
        if self.hidden_size % self.num_heads != 0:
            raise ValueError(
                f"hidden_size ({self.hidden_size}) must be divisible by "
                f"num_heads ({self.num_heads})"
            )
        head_dim = self.hidden_size // self.num_heads
        if self.ffn_hidden_size is None:
            self.ffn_hidden_size = 4 * self.hidden_size
        if self.rotary_dim is None:
            self.rotary_dim = head_dim
        if self.num_query_groups is None:
            self.num_query_groups = self.num_heads
        # Modules are always built in fp32; callers cast afterwards (as the
        # reference's benchmarks do with ``model.to(torch.bfloat16)``).
        self.dtype = torch.float32

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


def gpt_preset(name: str, **overrides) -> ReferenceGPTConfig:
    """GPT-2-style configs behind the names 345M / 760M / 1.3B.

    GELU MLP, learned positions, biases, fused QKV, vocab 50304: the knobs that
    make the parameter counts come out at 355.9M / 760.4M / 1315.8M.
    """
    table = {
        "tiny": dict(num_layers=2, hidden_size=64, num_heads=4, vocab_size=128, max_seq_len=32),
        "small": dict(num_layers=4, hidden_size=256, num_heads=4, vocab_size=1024, max_seq_len=256),
        "345m": dict(num_layers=24, hidden_size=1024, num_heads=16),
        "760m": dict(num_layers=24, hidden_size=1536, num_heads=16),
        "1.3b": dict(num_layers=24, hidden_size=2048, num_heads=16),
    }
    key = name.lower()
    if key not in table:
        raise ValueError(f"unknown GPT preset {name!r}; choose from {sorted(table)}")
    kw = dict(
        vocab_size=50304,
        max_seq_len=2048,
        use_bias=True,
        tie_word_embeddings=True,
        position_embedding_type="learned_absolute",
        activation_func="gelu",
        gated_linear_unit=False,
        use_fused_qkv=True,
    )
    kw.update(table[key])
    kw.update(overrides)
    return ReferenceGPTConfig(**kw)

"""Single-device oracle GPT (same names and op order as
nano_megatron/reference/model.py:12-110 of the reference)."""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch import Tensor, nn

from .config import ReferenceGPTConfig
from .layers import TransformerBlock, layer_norm, rms_norm


class ReferenceGPT(nn.Module):
    def __init__(self, config: ReferenceGPTConfig) -> None:
        super().__init__()
        self.config = config
        self.tok_emb = nn.Embedding(config.vocab_size, config.hidden_size)
        self.pos_emb = (
            nn.Embedding(config.max_seq_len, config.hidden_size)
            if config.position_embedding_type == "learned_absolute"
            else None
        )
        self.blocks = nn.ModuleList(TransformerBlock(config) for _ in range(config.num_layers))
        self.ln_f_weight = nn.Parameter(torch.ones(config.hidden_size))
        self.ln_f_bias = nn.Parameter(torch.zeros(config.hidden_size))
        self.layernorm_eps = config.layernorm_eps
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.tok_emb.weight
        self.to(dtype=torch.float32)

    def forward(self, input_ids: Tensor, positions: Optional[Tensor] = None) -> Tensor:
        return self._run(input_ids, positions, False)[0]

    def forward_with_activations(self, input_ids: Tensor, positions: Optional[Tensor] = None):
        return self._run(input_ids, positions, True)

    def _run(self, input_ids: Tensor, positions: Optional[Tensor], keep: bool) -> tuple[Tensor, dict[str, Any]]:
        batch, seq_len = input_ids.shape
        if seq_len > self.config.max_seq_len:
            raise ValueError(f"seq_len ({seq_len}) exceeds max_seq_len ({self.config.max_seq_len})")
        if positions is None:
            positions = torch.arange(seq_len, device=input_ids.device).unsqueeze(0).expand(batch, -1)
        emb = self.tok_emb(input_ids)
        if self.pos_emb is not None:
            emb = emb + self.pos_emb(positions)
        x = emb
        per_layer: list[dict[str, Any]] = []
        for block in self.blocks:
            if keep:
                x, acts = block(x, positions=positions, return_activations=True)
                per_layer.append(acts)
            else:
                x = block(x, positions=positions)
        if self.config.normalization == "rmsnorm":
            final_ln = rms_norm(x, self.ln_f_weight, self.layernorm_eps)
        else:
            final_ln = layer_norm(x, self.ln_f_weight, self.ln_f_bias, self.layernorm_eps)
        logits = self.lm_head(final_ln)
        if not keep:
            return logits, {}
        return logits, {"emb": emb, "layers": per_layer, "final_ln": final_ln, "logits": logits}

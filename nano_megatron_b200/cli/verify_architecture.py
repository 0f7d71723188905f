"""Architecture check: is a ``ReferenceGPTConfig`` the Megatron-LM GPT it claims to be?

Counterpart of the reference's ``scripts/verify_architecture.py:1-166``, which
prints a side-by-side table of a nano config and a Megatron-LM
``TransformerConfig`` and then runs one forward pass.  That script needs a
Megatron-LM checkout at a fixed path; this one works without it (the Megatron
side of the table is then the documented default of each field) and uses the
checkout when ``--megatron-path`` points at one.  It also *checks* instead of
only printing: parameter count against the closed-form count of the
architecture, the per-component knobs, and a forward pass on a reduced copy.

    python -m nano_megatron_b200.cli.verify_architecture --preset 345m [--knobs published]
"""
from __future__ import annotations

import argparse
import sys
from typing import Any, Optional

import torch

from ..reference import ReferenceGPT, ReferenceGPTConfig, gpt_preset

#: nano field -> (Megatron-LM TransformerConfig field, how to read the nano value)
FIELD_MAP = [
    ("num_layers", "num_layers", lambda c: c.num_layers),
    ("hidden_size", "hidden_size", lambda c: c.hidden_size),
    ("num_heads", "num_attention_heads", lambda c: c.num_heads),
    ("ffn_hidden_size", "ffn_hidden_size", lambda c: c.ffn_hidden_size),
    ("rotary_dim / head dim", "kv_channels", lambda c: c.hidden_size // c.num_heads),
    ("num_query_groups", "num_query_groups", lambda c: c.num_query_groups),
    ("layernorm_eps", "layernorm_epsilon", lambda c: c.layernorm_eps),
    ("use_bias", "add_bias_linear", lambda c: c.use_bias),
    ("gated_linear_unit", "gated_linear_unit", lambda c: c.gated_linear_unit),
    ("normalization", "normalization", lambda c: {"layernorm": "LayerNorm", "rmsnorm": "RMSNorm"}[c.normalization]),
    ("hidden_dropout", "hidden_dropout", lambda c: c.hidden_dropout),
    ("attention_dropout", "attention_dropout", lambda c: c.attention_dropout),
]


def expected_parameter_count(cfg: ReferenceGPTConfig) -> int:
    """Closed-form parameter count of the decoder described by ``cfg``."""
    h, f, v, layers = cfg.hidden_size, cfg.ffn_hidden_size, cfg.vocab_size, cfg.num_layers
    d = h // cfg.num_heads
    kv = cfg.num_query_groups * d
    bias = 1 if cfg.use_bias else 0
    attn = h * (h + 2 * kv) + bias * (h + 2 * kv) + h * h + bias * h
    fc1_out = 2 * f if cfg.gated_linear_unit else f
    mlp = h * fc1_out + bias * fc1_out + f * h + bias * h
    norms = 4 * h                                   # ln1 / ln2 weight + bias (bias kept in RMSNorm mode too)
    total = layers * (attn + mlp + norms) + 2 * h   # + final norm
    total += v * h                                  # token embedding
    if cfg.position_embedding_type == "learned_absolute":
        total += cfg.max_seq_len * h
    if not cfg.tie_word_embeddings:
        total += v * h                              # LM head
    return total


def count_parameters(cfg: ReferenceGPTConfig) -> int:
    with torch.device("meta"):
        model = ReferenceGPT(cfg)
    seen, total = set(), 0
    for p in model.parameters():
        if id(p) not in seen:
            seen.add(id(p))
            total += p.numel()
    return total


def megatron_side(cfg: ReferenceGPTConfig, megatron_path: Optional[str]) -> dict[str, Any]:
    """The matching Megatron-LM ``TransformerConfig`` values: read from a real
    ``TransformerConfig`` when a checkout is importable, else restated."""
    want = {m: get(cfg) for _, m, get in FIELD_MAP}
    if megatron_path:
        sys.path.insert(0, megatron_path)
        try:
            from megatron.core.transformer.transformer_config import TransformerConfig  # type: ignore
            tc = TransformerConfig(
                num_layers=cfg.num_layers, hidden_size=cfg.hidden_size, num_attention_heads=cfg.num_heads,
                ffn_hidden_size=cfg.ffn_hidden_size, kv_channels=cfg.hidden_size // cfg.num_heads,
                num_query_groups=cfg.num_query_groups, layernorm_epsilon=cfg.layernorm_eps,
                add_bias_linear=cfg.use_bias, gated_linear_unit=cfg.gated_linear_unit,
                normalization=want["normalization"], hidden_dropout=cfg.hidden_dropout,
                attention_dropout=cfg.attention_dropout)
            return {m: getattr(tc, m) for _, m, _ in FIELD_MAP}
        except Exception as exc:  # no checkout, or an incompatible one
            print(f"(Megatron-LM not usable from {megatron_path}: {type(exc).__name__}: {exc}; "
                  "using the restated values)")
    return want


def verify(cfg: ReferenceGPTConfig, megatron_path: Optional[str] = None, *, forward: bool = True,
           out=sys.stdout) -> bool:
    ok = True
    theirs = megatron_side(cfg, megatron_path)
    print(f"{'nano field':<24} {'Megatron-LM field':<22} {'nano':<12} {'Megatron-LM':<12}", file=out)
    print("-" * 72, file=out)
    for nano_name, meg_name, get in FIELD_MAP:
        mine = get(cfg)
        same = mine == theirs[meg_name]
        ok &= same
        print(f"{nano_name:<24} {meg_name:<22} {str(mine):<12} {str(theirs[meg_name]):<12} {'' if same else '<- differs'}",
              file=out)
    counted, expected = count_parameters(cfg), expected_parameter_count(cfg)
    print(f"\nparameters: {counted:,} (closed form {expected:,})", file=out)
    ok &= counted == expected
    print(f"position embedding : {'RoPE' if cfg.position_embedding_type == 'rope' else 'learned absolute'}", file=out)
    print(f"MLP activation     : {'SwiGLU' if cfg.gated_linear_unit else 'GELU (erf)'}", file=out)
    print(f"linear bias        : {'on' if cfg.use_bias else 'off'}", file=out)
    print(f"normalization      : {cfg.normalization}", file=out)
    print(f"QKV projection     : {'fused' if cfg.use_fused_qkv else 'separate'}", file=out)
    print(f"attention          : {'GQA, ' + str(cfg.num_query_groups) + ' groups' if cfg.num_query_groups < cfg.num_heads else 'MHA'}",
          file=out)
    print(f"embeddings         : {'tied' if cfg.tie_word_embeddings else 'untied'}", file=out)
    if forward:
        # one forward pass on a two-layer, narrow copy of the same architecture
        small = ReferenceGPTConfig(**{**cfg.__dict__, "num_layers": 2, "hidden_size": 8 * cfg.num_heads,
                                      "ffn_hidden_size": 32 * cfg.num_heads, "vocab_size": 256,
                                      "max_seq_len": min(cfg.max_seq_len, 64), "rotary_dim": None,
                                      "attn_backend": "unfused"})
        ids = torch.randint(0, small.vocab_size, (2, min(small.max_seq_len, 32)))
        with torch.no_grad():
            logits = ReferenceGPT(small)(ids)
        good = tuple(logits.shape) == (2, ids.shape[1], small.vocab_size) and bool(torch.isfinite(logits).all())
        print(f"forward pass       : logits {tuple(logits.shape)} {'ok' if good else 'BAD'}", file=out)
        ok &= good
    print("\narchitecture " + ("matches" if ok else "DOES NOT match"), file=out)
    return ok


def main(argv: Optional[list[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--preset", default="345m", choices=["345m", "760m", "1.3b", "small"])
    ap.add_argument("--knobs", default="gpt2", choices=["gpt2", "published"],
                    help="published: RoPE, SwiGLU, no bias, untied, vocabulary 51200 (the reference's benchmark knobs)")
    ap.add_argument("--megatron-path", default=None, help="a Megatron-LM checkout to read TransformerConfig from")
    ap.add_argument("--no-forward", action="store_true")
    args = ap.parse_args(argv)
    over = {}
    if args.knobs == "published":
        over = dict(vocab_size=51200, use_bias=False, tie_word_embeddings=False, position_embedding_type="rope",
                    activation_func="swiglu", gated_linear_unit=True)
    cfg = gpt_preset(args.preset, attn_backend="unfused", **over)
    return 0 if verify(cfg, args.megatron_path, forward=not args.no_forward) else 1


if __name__ == "__main__":
    sys.exit(main())

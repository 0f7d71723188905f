"""Single-device oracle run: seed, build, one random batch, N optimizer steps,
save the per-step trajectory.

Counterpart of scripts/run_reference_gpt.py:22-108 of the reference, with the
architecture knobs that script cannot express (GELU vs SwiGLU, learned vs rotary
positions, tied embeddings, bias) exposed as flags.  As there, the batch is
drawn *after* the model is built from the same seed.

    python -m nano_megatron_b200.cli.run_reference_gpt --layers 2 --hidden 64 --heads 4 \
        --vocab 128 --seq 32 --batch 2 --gelu --learned-pos --tied --steps 3 --out traj.pt
"""
from __future__ import annotations

import argparse
import sys

import torch

from ..reference import AdamW, ReferenceGPT, ReferenceGPTConfig, reference_train_loop, seed_all


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--device", default="cpu")
    p.add_argument("--out", default=None)
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--hidden", type=int, default=64)
    p.add_argument("--heads", type=int, default=4)
    p.add_argument("--ffn", type=int, default=None)
    p.add_argument("--vocab", type=int, default=128)
    p.add_argument("--seq", type=int, default=32)
    p.add_argument("--batch", type=int, default=2)
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--weight-decay", type=float, default=0.01)
    p.add_argument("--gelu", action="store_true", help="GELU MLP instead of SwiGLU")
    p.add_argument("--learned-pos", action="store_true", help="learned absolute positions instead of RoPE")
    p.add_argument("--tied", action="store_true", help="tie input and output embeddings")
    p.add_argument("--bias", action="store_true")
    p.add_argument("--fused-qkv", action="store_true")
    p.add_argument("--capture", default="full", choices=["minimal", "grads", "full"])
    return p


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    seed_all(args.seed)
    cfg = ReferenceGPTConfig(
        vocab_size=args.vocab, max_seq_len=args.seq, hidden_size=args.hidden, num_layers=args.layers,
        num_heads=args.heads, ffn_hidden_size=args.ffn, use_bias=args.bias, tie_word_embeddings=args.tied,
        position_embedding_type="learned_absolute" if args.learned_pos else "rope",
        gated_linear_unit=not args.gelu, activation_func="gelu" if args.gelu else "swiglu",
        use_fused_qkv=args.fused_qkv, attn_backend="unfused")
    device = torch.device(args.device)
    model = ReferenceGPT(cfg).to(device)
    opt = AdamW(model.named_parameters(), lr=args.lr, weight_decay=args.weight_decay)
    ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq), device=device)
    results = reference_train_loop(model, opt, [ids], steps=args.steps, capture_level=args.capture)
    for r in results:
        print(f"step {r.step}: loss {r.loss.item():.6f}")
    if args.out:
        torch.save([{"step": r.step, "loss": r.loss, "logits": r.logits, "params": r.params, "grads": r.grads,
                     "activations": r.activations, "optimizer_state": r.optimizer_state} for r in results], args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Merge a sharded checkpoint into one file in the single-device layout.

    python -m nano_megatron_b200.cli.merge_checkpoint CKPT_DIR OUT.pt

``CKPT_DIR`` holds the ``shard_tp*_pp*.pt`` files written by
``nano_megatron_b200.utils.save_checkpoint``; ``OUT.pt`` receives
``{"config": dict, "step": int, "model": state_dict, "optimizer": state}`` where
``model`` loads into ``ReferenceGPT(ReferenceGPTConfig(**config))`` with the
parameter names of nano_megatron/reference/model.py and ``optimizer`` is the
``{name: {"exp_avg", "exp_avg_sq", "step"}}`` form of
nano_megatron/reference/optimizer.py:104-131.  The reference itself has no
sharded checkpoints and hence no such tool.
"""
from __future__ import annotations

import argparse
import dataclasses
import sys

import torch

from ..utils.checkpoint import merge_checkpoint


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("directory")
    ap.add_argument("output")
    args = ap.parse_args(argv)
    merged = merge_checkpoint(args.directory)
    cfg = dataclasses.asdict(merged["config"])
    cfg.pop("dtype", None)   # a torch.dtype default; not part of the portable description
    torch.save({"config": cfg, "step": merged["step"], "model": merged["model"], "optimizer": merged["optimizer"]},
               args.output)
    n_params = sum(t.numel() for n, t in merged["model"].items()
                   if not (n == "lm_head.weight" and cfg.get("tie_word_embeddings")))
    print(f"merged step {merged['step']}: {len(merged['model'])} tensors, {n_params} parameters -> {args.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Sharded checkpoints with the reference's parameter names.

The reference has no on-disk model format (only ``AdamW.state_dict`` and a
trajectory dump, nano_megatron/reference/optimizer.py:104-131,
scripts/run_reference_gpt.py:99-103).  Here every (tp, pp) coordinate with
``dp_rank == cp_rank == 0`` writes one file ``shard_tp{t}_pp{p}.pt`` holding its
local tensors under their *reference* names (pipeline stages re-index
``blocks.{local}`` to the global layer), the optimizer state in the
reference's ``{name: {exp_avg, exp_avg_sq, step}}`` form, the step counter and
the RNG state.  ``merge_checkpoint`` is the inverse of the TP shard rules
(contiguous row blocks for column/vocab layers, per-block shards for fused QKV
and gated fc1, column blocks for row layers, replicated otherwise) and returns a
full ``ReferenceGPT.state_dict()``; ``load_checkpoint`` re-shards a merged state
for any other TP/PP layout.
"""
from __future__ import annotations

import glob
import os
import re
from typing import Any, Optional

import torch
from torch import Tensor, nn

from ..reference.config import ReferenceGPTConfig

_COLUMN = ("q_proj", "k_proj", "v_proj", "lm_head", "tok_emb")


def _kind(name: str, cfg: ReferenceGPTConfig) -> str:
    leaf = name.rsplit(".", 1)[-1]
    if "qkv_proj" in name:
        return "qkv"
    if "fc1" in name:
        return "gated" if cfg.gated_linear_unit else "column"
    if any(k in name for k in _COLUMN):
        return "column"
    if ("out_proj" in name or "fc2" in name) and leaf == "weight":
        return "row"
    return "replicated"


def _blocks(name: str, cfg: ReferenceGPTConfig) -> Optional[tuple[int, ...]]:
    d = cfg.hidden_size // cfg.num_heads
    kind = _kind(name, cfg)
    if kind == "qkv":
        kv = cfg.num_query_groups * d
        return (cfg.hidden_size, kv, kv)
    if kind == "gated":
        return (cfg.ffn_hidden_size, cfg.ffn_hidden_size)
    return None


def shard_tensor(name: str, full: Tensor, cfg: ReferenceGPTConfig, tp_rank: int, tp_size: int) -> Tensor:
    """The slice of a full reference tensor that TP rank ``tp_rank`` of ``tp_size`` owns."""
    if tp_size == 1:
        return full
    kind = _kind(name, cfg)
    if kind in ("qkv", "gated"):
        parts, start = [], 0
        for size in _blocks(name, cfg):
            n = size // tp_size
            parts.append(full[start + tp_rank * n:start + (tp_rank + 1) * n])
            start += size
        return torch.cat(parts, dim=0)
    if kind == "column":
        n = full.shape[0] // tp_size
        return full[tp_rank * n:(tp_rank + 1) * n]
    if kind == "row":
        n = full.shape[1] // tp_size
        return full[:, tp_rank * n:(tp_rank + 1) * n]
    return full


def unshard_tensor(name: str, shards: list[Tensor], cfg: ReferenceGPTConfig) -> Tensor:
    """Inverse of :func:`shard_tensor` given the shards of all TP ranks in order."""
    if len(shards) == 1:
        return shards[0]
    kind = _kind(name, cfg)
    t = len(shards)
    if kind in ("qkv", "gated"):
        out, start = [], 0
        for size in _blocks(name, cfg):
            n = size // t
            out.extend(s[start:start + n] for s in shards)
            start += n
        return torch.cat(out, dim=0)
    if kind == "column":
        return torch.cat(shards, dim=0)
    if kind == "row":
        return torch.cat(shards, dim=1)
    return shards[0]


def _global_name(local: str, layer_offset: int) -> str:
    m = re.match(r"blocks\.(\d+)\.(.*)", local)
    if m:
        return f"blocks.{int(m.group(1)) + layer_offset}.{m.group(2)}"
    return local


def _local_name(global_name: str, layer_offset: int, layers_here: int) -> Optional[str]:
    m = re.match(r"blocks\.(\d+)\.(.*)", global_name)
    if m:
        idx = int(m.group(1)) - layer_offset
        return f"blocks.{idx}.{m.group(2)}" if 0 <= idx < layers_here else None
    return global_name


def save_checkpoint(directory: str, model: nn.Module, optimizer: Any, ctx: Any, *, step: int,
                    extra: Optional[dict] = None) -> Optional[str]:
    """Write this rank's shard (only ``dp_rank == cp_rank == 0`` ranks write).  Returns the path or None."""
    if ctx.data_parallel_rank != 0 or ctx.context_parallel_rank != 0:
        return None
    os.makedirs(directory, exist_ok=True)
    cfg: ReferenceGPTConfig = model.config
    per_stage = cfg.num_layers // ctx.pipeline_parallel_size
    offset = ctx.pipeline_parallel_rank * per_stage
    tensors = {_global_name(n, offset): p.detach().cpu().clone() for n, p in model.named_parameters()}
    opt_state = {}
    if optimizer is not None:
        opt_state = {_global_name(n, offset): {"exp_avg": e["exp_avg"].cpu(), "exp_avg_sq": e["exp_avg_sq"].cpu(),
                                               "step": int(e["step"])}
                     for n, e in optimizer.state_dict().items()}
    payload = {
        "format": "nano_megatron_b200/1",
        "config": dict(cfg.__dict__),
        "layout": {"tp": ctx.tensor_parallel_size, "pp": ctx.pipeline_parallel_size,
                   "tp_rank": ctx.tensor_parallel_rank, "pp_rank": ctx.pipeline_parallel_rank},
        "step": int(step),
        "model": tensors,
        "optimizer": opt_state,
        "rng": {"torch": torch.get_rng_state(),
                "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None},
        "extra": extra or {},
    }
    path = os.path.join(directory, f"shard_tp{ctx.tensor_parallel_rank}_pp{ctx.pipeline_parallel_rank}.pt")
    tmp = path + ".tmp"
    torch.save(payload, tmp)
    os.replace(tmp, path)                                  # atomic: a crash never leaves half a file
    return path


def merge_checkpoint(directory: str) -> dict[str, Any]:
    """Reassemble the full reference state: ``{"config", "step", "model", "optimizer"}``."""
    files = sorted(glob.glob(os.path.join(directory, "shard_tp*_pp*.pt")))
    if not files:
        raise FileNotFoundError(f"no checkpoint shards in {directory}")
    shards = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
    cfg_dict = dict(shards[0]["config"])
    cfg_dict.pop("dtype", None)
    cfg = ReferenceGPTConfig(**cfg_dict)
    tp = shards[0]["layout"]["tp"]
    by_name: dict[str, dict[int, Tensor]] = {}
    opt_by_name: dict[str, dict[int, dict]] = {}
    for sh in shards:
        r = sh["layout"]["tp_rank"]
        for n, t in sh["model"].items():
            by_name.setdefault(n, {})[r] = t
        for n, e in sh["optimizer"].items():
            opt_by_name.setdefault(n, {})[r] = e
    model = {n: unshard_tensor(n, [parts[r] for r in range(tp)], cfg) for n, parts in by_name.items()}
    if cfg.tie_word_embeddings and "tok_emb.weight" in model:
        model["lm_head.weight"] = model["tok_emb.weight"]
    optimizer = {}
    for n, parts in opt_by_name.items():
        optimizer[n] = {
            "exp_avg": unshard_tensor(n, [parts[r]["exp_avg"] for r in range(tp)], cfg),
            "exp_avg_sq": unshard_tensor(n, [parts[r]["exp_avg_sq"] for r in range(tp)], cfg),
            "step": parts[0]["step"],
        }
    return {"config": cfg, "step": shards[0]["step"], "model": model, "optimizer": optimizer,
            "rng": shards[0]["rng"], "extra": shards[0].get("extra", {})}


def load_checkpoint(directory: str, model: nn.Module, optimizer: Any, ctx: Any, *, restore_rng: bool = False) -> int:
    """Load (re-sharding for this rank's layout) and return the saved step."""
    merged = merge_checkpoint(directory)
    cfg: ReferenceGPTConfig = model.config
    per_stage = cfg.num_layers // ctx.pipeline_parallel_size
    offset = ctx.pipeline_parallel_rank * per_stage
    t, r = ctx.tensor_parallel_size, ctx.tensor_parallel_rank
    with torch.no_grad():
        for n, p in model.named_parameters():
            full = merged["model"][_global_name(n, offset)]
            p.copy_(shard_tensor(_global_name(n, offset), full, cfg, r, t).to(device=p.device, dtype=p.dtype))
    if optimizer is not None and merged["optimizer"]:
        state = {}
        for n, _ in model.named_parameters():
            g = _global_name(n, offset)
            if g in merged["optimizer"]:
                e = merged["optimizer"][g]
                state[n] = {"exp_avg": shard_tensor(g, e["exp_avg"], cfg, r, t),
                            "exp_avg_sq": shard_tensor(g, e["exp_avg_sq"], cfg, r, t), "step": e["step"]}
        optimizer.load_state_dict(state)
    if restore_rng and merged.get("rng"):
        torch.set_rng_state(merged["rng"]["torch"])
        if merged["rng"].get("cuda") is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(merged["rng"]["cuda"])
    return int(merged["step"])

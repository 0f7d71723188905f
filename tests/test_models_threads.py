"""The real TP / SP / CP GPT on simulated ranks at sizes the socket-based suite
does not reach (TP 4, TP 4 + SP, CP 4, TP 2 x CP 2): logits, loss and every
parameter gradient against the single-device oracle on the same batch."""
from __future__ import annotations

import pytest
import torch

from nano_megatron_b200.distributed import DistributedDataParallel
from nano_megatron_b200.models import build_tp_gpt_from_reference

from ._thread_ranks import run_ranks, thread_context
from .test_distributed_gloo import _check_grads, _close, _model_cfg, _reference


@pytest.mark.parametrize("tp,sp,knobs", [
    (4, False, dict()),
    (4, True, dict()),
    (4, True, dict(position_embedding_type="learned_absolute", gated_linear_unit=False, use_fused_qkv=True,
                   tie_word_embeddings=True)),
    (4, False, dict(use_fused_qkv=True, num_query_groups=4, gated_linear_unit=True)),
])
def test_tensor_and_sequence_parallel_gpt_at_four_ranks(tp, sp, knobs):
    cfg = _model_cfg(**knobs)
    torch.manual_seed(1234)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    ref, ref_logits, ref_loss = _reference(cfg, ids)

    def prepare(rank, be):
        ctx = thread_context(rank, be, tp=tp, sequence_parallel=sp)
        return ctx, build_tp_gpt_from_reference(ref, ctx)

    def rank_fn(rank, be, prepared):
        ctx, model = prepared
        logits = model(ids)
        loss = model.shifted_cross_entropy(logits, ids)
        loss.backward()
        _close(loss.detach(), ref_loss, "loss")
        _check_grads(model, ref, ctx, cfg)
        return logits.detach()

    shards = run_ranks(tp, rank_fn, prepare)
    _close(torch.cat(shards, dim=-1), ref_logits, "logits")          # vocabulary shards side by side


@pytest.mark.parametrize("tp,cp", [(1, 4), (2, 2)])
def test_context_parallel_gpt(tp, cp):
    cfg = _model_cfg()
    torch.manual_seed(1234)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    labels = ids.clone()
    labels[0, 4] = -100
    ref, ref_logits, ref_loss = _reference(cfg, ids, labels)
    s_loc = 16 // cp

    def prepare(rank, be):
        ctx = thread_context(rank, be, tp=tp, cp=cp)
        return ctx, build_tp_gpt_from_reference(ref, ctx)

    def rank_fn(rank, be, prepared):
        ctx, model = prepared
        ddp = DistributedDataParallel(model, ctx)                     # collective (parameter broadcast): on the rank's thread
        logits = ddp(ids)
        assert logits.shape[1] == s_loc                               # only the local sequence shard
        loss = model.shifted_cross_entropy(logits, labels)
        loss.backward()
        ddp.finish_grad_sync()                                        # mean over the CP group
        _check_grads(model, ref, ctx, cfg)
        return ctx.tensor_parallel_rank, ctx.context_parallel_rank, logits.detach(), loss.detach()

    results = run_ranks(tp * cp, rank_fn, prepare)
    rows = []
    for c in range(cp):
        parts = sorted((r for r in results if r[1] == c), key=lambda r: r[0])
        rows.append(torch.cat([p[2] for p in parts], dim=-1))
    _close(torch.cat(rows, dim=1), ref_logits, "logits")
    mean = torch.stack([r[3] for r in results if r[0] == 0]).mean()   # CP-local means average to the global mean
    _close(mean, ref_loss, "loss")

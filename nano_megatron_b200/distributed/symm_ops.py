"""Operators that read or write peers' symmetric buffers from inside compute kernels."""
from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from .symm_mem import CHANNEL_CP, SymmetricWorkspace


class _KVExchange:
    """Per-workspace pool of symmetric K/V slots and one dK/dV staging area.

    A slot pair is leased by an attention call that will run a backward pass
    and stays taken until that backward has run (or its autograd graph is
    dropped): the backward re-reads K/V from the slot -- its own and, through
    peer pointers, the other ranks'.  Slots are handed out in call order and the
    order restarts with every forward pass when nothing is outstanding, so in
    the steady state every layer gets the same slot every step; with several
    forward passes outstanding (microbatches, an evaluation pass between
    forward and backward) later passes get further slots instead of overwriting
    K/V that a pending backward still needs.  All ranks of the group make the
    same calls in the same order, so their slot choices agree.
    """

    def __init__(self, ws: SymmetricWorkspace) -> None:
        self.ws = ws
        self.slots: list[tuple[Tensor, Tensor]] = []
        self.leased: list[bool] = []
        self.cursor = 0
        self.staging: dict[tuple, tuple[Tensor, Tensor]] = {}

    def next_slot(self, like: Tensor, lease: bool) -> tuple[int, tuple[Tensor, Tensor]]:
        while self.cursor < len(self.slots) and self.leased[self.cursor]:
            self.cursor += 1
        if self.cursor == len(self.slots):
            k = self.ws.alloc_tensor(like.numel(), like.dtype).view(like.shape)
            v = self.ws.alloc_tensor(like.numel(), like.dtype).view(like.shape)
            self.slots.append((k, v))
            self.leased.append(False)
        index = self.cursor
        pair = self.slots[index]
        if pair[0].shape != like.shape:
            raise RuntimeError("context-parallel K/V shape changed between steps")
        self.leased[index] = lease
        self.cursor += 1
        return index, pair

    def next_packed(self, like: Tensor, lease: bool) -> tuple[int, Tensor]:
        """Like ``next_slot`` for ONE buffer of ``like``'s shape (a packed QKV output)."""
        while self.cursor < len(self.slots) and self.leased[self.cursor]:
            self.cursor += 1
        if self.cursor == len(self.slots):
            buf = self.ws.alloc_tensor(like.numel(), like.dtype).view(like.shape)
            self.slots.append((buf, buf))
            self.leased.append(False)
        index = self.cursor
        buf = self.slots[index][0]
        if buf.shape != like.shape:
            raise RuntimeError("context-parallel QKV shape changed between steps")
        self.leased[index] = lease
        self.cursor += 1
        return index, buf

    def release(self, index: int) -> None:
        self.leased[index] = False

    def stage(self, like: Tensor) -> tuple[Tensor, Tensor]:
        """dK / dV staging ``[size, *like.shape]``, two pairs used alternately: a
        rank may already store the next layer's tiles into a peer's staging while
        that peer still sums the previous layer's."""
        key = (tuple(like.shape), like.dtype)
        if key not in self.staging:
            n = self.ws.size * like.numel()
            pairs = []
            for _ in range(2):
                dk = self.ws.alloc_tensor(n, like.dtype).view(self.ws.size, *like.shape)
                dv = self.ws.alloc_tensor(n, like.dtype).view(self.ws.size, *like.shape)
                pairs.append((dk, dv))
            self.staging[key] = [pairs, 0]
        pairs, turn = self.staging[key]
        self.staging[key][1] = turn ^ 1
        return pairs[turn]


class _SlotLease:
    """Gives a K/V slot back when the attention call's autograd context goes away."""

    def __init__(self, ex: _KVExchange, index: int) -> None:
        self.ex, self.index = ex, index

    def release(self) -> None:
        if self.ex is not None:
            self.ex.release(self.index)
            self.ex = None

    def __del__(self) -> None:
        self.release()


def _exchange(ws: SymmetricWorkspace) -> _KVExchange:
    ex = getattr(ws, "_kv_exchange", None)
    if ex is None:
        ex = _KVExchange(ws)
        ws._kv_exchange = ex
    return ex


def begin_step(ws: SymmetricWorkspace) -> None:
    """Restart the K/V slot order (called at the start of every forward pass);
    slots still leased by a pending backward are skipped."""
    _exchange(ws).cursor = 0


class _CPFlashPeer(torch.autograd.Function):
    """Context-parallel attention whose kernel reads the peers' K/V in place.

    forward : K/V must be peer-addressable.  When the projection wrote them
              straight into symmetric memory (``qkv_slot``) they are used where
              they are; otherwise they are copied into a leased slot.  One
              barrier (every rank's K/V is published), then ONE attention launch
              whose TMA loads fetch chunk c from rank c's memory.
    backward: ONE attention launch computes dQ and this rank's dK/dV contribution
              to every visible chunk, storing chunk c's tiles straight into slot
              [my_rank] of rank c's staging buffer; then ONE launch on every rank
              meets the group in a flag round and sums the slots of the ranks
              that can see this rank's shard (rank >= own), un-rotating dK when
              the projection applied rotary embeddings.
    """

    @staticmethod
    def forward(ctx: Any, q: Tensor, k: Tensor, v: Tensor, scale: float, ws: SymmetricWorkspace, cp_rank: int,
                cp_size: int, lease: Any = None, rope: Any = None):
        from ..ops.attention import attn_fwd

        ex = _exchange(ws)
        if ws.contains(k) and ws.contains(v):
            k_slot, v_slot = k, v                    # already in symmetric memory (leased by the caller)
        else:
            # Inside a CUDA graph capture forward and backward of the step are recorded
            # together and replayed as a unit: nothing stays outstanding, no lease.
            take = any(ctx.needs_input_grad[:3]) and not torch.cuda.is_current_stream_capturing()
            k, v = k.contiguous(), v.contiguous()
            index, (k_slot, v_slot) = ex.next_slot(k, lease=take)
            lease = _SlotLease(ex, index) if take else None
            k_slot.copy_(k)
            v_slot.copy_(v)
        ctx.lease = lease
        ws.barrier(CHANNEL_CP)                       # every rank's K/V is published
        ks = [ws.peer_strided(k_slot, r) for r in range(cp_size)]
        vs = [ws.peer_strided(v_slot, r) for r in range(cp_size)]
        out, lse = attn_fwd(q, ks, vs, scale, q_pos0=cp_rank * q.shape[1])
        ctx.save_for_backward(q, out, lse)
        ctx.kv = (k_slot, v_slot)
        ctx.meta = (scale, ws, cp_rank, cp_size, rope)
        return out

    @staticmethod
    def backward(ctx: Any, dout: Tensor):
        from ..ops.attention import attn_bwd

        q, out, lse = ctx.saved_tensors
        k_slot, v_slot = ctx.kv
        scale, ws, cp_rank, cp_size, rope = ctx.meta
        ex = _exchange(ws)
        like = torch.empty(k_slot.shape, dtype=k_slot.dtype, device="meta")
        dk_stage, dv_stage = ex.stage(like)
        ks = [ws.peer_strided(k_slot, r) for r in range(cp_size)]
        vs = [ws.peer_strided(v_slot, r) for r in range(cp_size)]
        # chunk c's gradient tiles go to slot [cp_rank] of rank c's staging buffer
        dks = [ws.peer_view(dk_stage, r)[cp_rank] for r in range(cp_size)]
        dvs = [ws.peer_view(dv_stage, r)[cp_rank] for r in range(cp_size)]
        # dq, dk and dv are slices of ONE packed gradient, as the projection's backward wants it
        b, s, hq, d = q.shape
        hkv = k_slot.shape[2]
        dqkv = torch.empty((b, s, (hq + 2 * hkv) * d), dtype=q.dtype, device=q.device)
        dq = dqkv[..., : hq * d].view(b, s, hq, d)
        dk = dqkv[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
        dv = dqkv[..., (hq + hkv) * d:].view(b, s, hkv, d)
        attn_bwd(q, ks, vs, out, dout, lse, scale, q_pos0=cp_rank * s, dk_chunks=dks, dv_chunks=dvs, dq=dq, rope=rope)
        # flag round + sum of the contributions (+ inverse rotation of dK) in one launch
        ws.cp_dkv_reduce(dk_stage, dv_stage, dk, dv, cp_rank, rope=rope)
        if ctx.lease is not None:
            ctx.lease.release()
        return dq, dk, dv, None, None, None, None, None, None


def cp_flash_attention_peer(q: Tensor, k: Tensor, v: Tensor, scale: float, ws: SymmetricWorkspace, cp_rank: int,
                            cp_size: int, lease: Any = None, rope: Any = None) -> Tensor:
    """``rope``: q and k were rotated by the projection's epilogue; the backward
    returns un-rotated dq / dk (see ``flash_attention_packed``)."""
    return _CPFlashPeer.apply(q, k, v, float(scale), ws, cp_rank, cp_size, lease, rope)


def lease_packed_slot(ws: SymmetricWorkspace, shape: tuple, dtype: torch.dtype, will_backward: bool):
    """A symmetric buffer for a packed QKV projection output (the K and V slices
    of it are what the peers read), leased until the attention's backward has
    run.  Returns ``(buffer, lease or None)``."""
    ex = _exchange(ws)
    take = will_backward and not torch.cuda.is_current_stream_capturing()
    like = torch.empty(shape, dtype=dtype, device="meta")
    index, buf = ex.next_packed(like, lease=take)
    return buf, (_SlotLease(ex, index) if take else None)


class _SPEmbeddingFn(torch.autograd.Function):
    """Vocabulary-parallel embedding whose output is sequence-sharded.

    The reference all-reduces the masked lookups of all ranks and then narrows
    to the local sequence shard (nano_megatron/model/tp_gpt.py:546-561).  Each
    row has exactly one non-zero contributor, so no arithmetic is needed: the
    rank that owns a token's vocabulary id writes the row (token + position
    embedding) directly into the buffer of the rank that owns its sequence
    position.  Backward gathers the gradient shards and scatter-adds the rows of
    this rank's vocabulary shard.
    """

    @staticmethod
    def forward(ctx: Any, ids: Tensor, positions, tok_w: Tensor, pos_w, vocab_start: int, ws: SymmetricWorkspace,
                site: Any):
        b, s = ids.shape
        h = tok_w.shape[1]
        rows = b * s // ws.size
        # one buffer per shape: the result is copied out below, and every rank
        # passes the leading barrier only when all are done with the previous use
        cache = ws.__dict__.setdefault("_emb_out", {})
        key = ("sp", rows, h)
        if key not in cache:
            cache[key] = ws.alloc_tensor(rows * h, tok_w.dtype).view(rows, h)
        out = cache[key]
        ids_c = ids.contiguous()
        pos_c = positions.contiguous() if positions is not None else None
        ws.barrier()                      # every rank is done with the previous step's output
        ws.embedding_scatter(ids_c, pos_c, tok_w, pos_w, out, vocab_start, s)
        ws.barrier()                      # every row of my shard has been written
        ctx.save_for_backward(ids_c, pos_c)
        ctx.meta = (tok_w, pos_w, vocab_start, ws, (b, s, h))
        return out.view(b, s // ws.size, h).clone()

    @staticmethod
    def backward(ctx: Any, dy: Tensor):
        from ..ops import kernels

        ids, positions = ctx.saved_tensors
        tok_w, pos_w, vocab_start, ws, (b, s, h) = ctx.meta
        width = s // ws.size
        shards = ws.all_gather(dy.contiguous())                       # [ranks, B, S/t, H]
        full = shards.permute(1, 0, 2, 3).reshape(b, s, h).contiguous()
        results = []
        for param in (tok_w, pos_w):
            if param is None:
                results.append((None, None))
                continue
            # sequence-parallel replicated parameters must go through autograd so that
            # their TP gradient hook runs
            main = None if getattr(param, "_nmb_sp_replicated", False) else getattr(param, "main_grad", None)
            results.append((main if main is not None else torch.zeros_like(param), main is not None))
        d_tok, tok_direct = results[0]
        d_pos, pos_direct = results[1]
        kernels.embedding_bwd(ids, None, full, d_tok, None, vocab_start)
        if d_pos is not None:
            # Position rows: only this rank's sequence shard, i.e. a partial sum that
            # the sequence-parallel gradient hook completes over the TP group.
            lo = ws.rank * width
            kernels.embedding_bwd(ids[:, lo:lo + width].contiguous(), positions[:, lo:lo + width].contiguous(),
                                  dy.contiguous(), None, d_pos, vocab_start)
        for param, direct in ((tok_w, tok_direct), (pos_w, pos_direct)):
            if param is not None and direct:
                from ..ops.functional import note_grad_write
                note_grad_write(param, False)   # scatter-add into the gradient buffer
                ready = getattr(param, "_nmb_grad_ready", None)
                if ready is not None:
                    ready()
        return (None, None, None if tok_direct else d_tok, None if (pos_w is None or pos_direct) else d_pos,
                None, None, None)


def sp_embedding(ids: Tensor, positions, tok_w: Tensor, pos_w, vocab_start: int, ws: SymmetricWorkspace,
                 site: Any) -> Tensor:
    return _SPEmbeddingFn.apply(ids, positions, tok_w, pos_w, vocab_start, ws, site)


class _TPEmbeddingFn(torch.autograd.Function):
    """Vocabulary-parallel embedding with a replicated ``[B, S, H]`` output
    (tensor parallelism without sequence parallelism).

    The reference sums the ranks' masked lookups with an all-reduce
    (nano_megatron/parallel/vocab_parallel.py:86-100).  Every row has exactly one
    non-zero contributor, so the owner of a token's vocabulary id writes the row
    (token + position embedding) into every rank's buffer instead -- no
    arithmetic, one pass.  Backward is local: the output gradient is replicated
    and each rank scatter-adds the rows of its own vocabulary shard.
    """

    @staticmethod
    def forward(ctx: Any, ids: Tensor, positions, tok_w: Tensor, pos_w, vocab_start: int, ws: SymmetricWorkspace):
        b, s = ids.shape
        h = tok_w.shape[1]
        cache = ws.__dict__.setdefault("_emb_out", {})
        key = ("all", b * s, h)
        if key not in cache:
            cache[key] = ws.alloc_tensor(b * s * h, tok_w.dtype).view(b * s, h)
        out = cache[key]
        ids_c = ids.contiguous()
        pos_c = positions.contiguous() if positions is not None else None
        ws.barrier()                      # every rank has copied the previous result out
        ws.embedding_scatter(ids_c, pos_c, tok_w, pos_w, out, vocab_start, s, to_all=True)
        ws.barrier()                      # every row has been written by its owner
        ctx.save_for_backward(ids_c, pos_c)
        ctx.params = (tok_w, pos_w)
        ctx.vocab_start = vocab_start
        return out.view(b, s, h).clone()

    @staticmethod
    def backward(ctx: Any, dy: Tensor):
        from ..ops.functional import _EmbeddingFn
        return (*_EmbeddingFn.backward(ctx, dy), None)


def tp_embedding(ids: Tensor, positions, tok_w: Tensor, pos_w, vocab_start: int, ws: SymmetricWorkspace) -> Tensor:
    return _TPEmbeddingFn.apply(ids, positions if pos_w is not None else None, tok_w, pos_w, vocab_start, ws)

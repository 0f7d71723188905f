"""Attention backend selection and the unfused / merge arithmetic on CPU."""
from __future__ import annotations

import math

import pytest
import torch

import nano_megatron_b200.parallel as P
from nano_megatron_b200.parallel import attention_backend as AB

CPU = torch.device("cpu")


def _dense_causal(q, k, v, scale, query_start=0):
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * scale
    qpos = torch.arange(query_start, query_start + q.size(2))[:, None]
    kpos = torch.arange(k.size(2))[None, :]
    return torch.softmax(s.masked_fill(kpos > qpos, float("-inf")), dim=-1) @ v


# ------------------------------------------------------------- resolution --
@pytest.mark.parametrize("requested,dtype,want", [("unfused", torch.bfloat16, "unfused"),
                                                  ("auto", torch.float32, "unfused"),
                                                  ("auto", torch.bfloat16, "unfused")])   # CPU never gets flash
def test_resolution_on_cpu(requested, dtype, want):
    assert P.resolve_attention_backend(requested=requested, dtype=dtype, device=CPU) == want


def test_asking_for_activations_forces_the_unfused_path_before_any_check():
    assert P.resolve_attention_backend(requested="flash", dtype=torch.float32, device=CPU,
                                       return_activations=True) == "unfused"
    assert P.resolve_attention_backend(requested="nonsense", dtype=torch.float32, device=CPU,
                                       return_activations=True) == "unfused"


def test_flash_is_a_hard_requirement_when_named():
    with pytest.raises(RuntimeError, match="device must be CUDA"):
        P.resolve_attention_backend(requested="flash", dtype=torch.bfloat16, device=CPU)
    with pytest.raises(RuntimeError, match="dtype must be bfloat16"):
        P.resolve_attention_backend(requested="flash", dtype=torch.float32, device=CPU)
    with pytest.raises(ValueError, match="requested must be one of"):
        P.resolve_attention_backend(requested="fused", dtype=torch.bfloat16, device=CPU)


def test_auto_picks_flash_for_bf16_on_cuda_when_the_library_is_built(monkeypatch):
    monkeypatch.setattr(AB, "flash_attn_available", lambda: True)
    assert P.resolve_attention_backend(requested="auto", dtype=torch.bfloat16, device=torch.device("cuda", 0)) == "flash"
    assert P.resolve_attention_backend(requested="auto", dtype=torch.float16, device=torch.device("cuda", 0)) == "unfused"
    monkeypatch.setattr(AB, "flash_attn_available", lambda: False)
    assert P.resolve_attention_backend(requested="auto", dtype=torch.bfloat16, device=torch.device("cuda", 0)) == "unfused"
    with pytest.raises(RuntimeError, match="not built"):
        P.resolve_attention_backend(requested="flash", dtype=torch.bfloat16, device=torch.device("cuda", 0))


# ---------------------------------------------------------------- unfused --
def test_unfused_matches_dense_softmax_and_supports_a_query_offset():
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 3, 8, 4) for _ in range(3))
    scale = 1 / math.sqrt(4)
    assert torch.allclose(P.unfused_causal_attention(q, k, v, scale=scale), _dense_causal(q, k, v, scale), atol=1e-6)
    tail = P.unfused_causal_attention(q[:, :, 4:], k, v, scale=scale, query_start=4)
    assert torch.allclose(tail, _dense_causal(q, k, v, scale)[:, :, 4:], atol=1e-6)


def test_unfused_argument_checks():
    q, k = torch.randn(1, 2, 4, 4), torch.randn(1, 2, 8, 4)
    with pytest.raises(ValueError, match="query_start is required"):
        P.unfused_causal_attention(q, k, k, scale=1.0)
    with pytest.raises(ValueError, match="exceeds"):
        P.unfused_causal_attention(q, k, k, scale=1.0, query_start=6)
    with pytest.raises(ValueError, match="4D"):
        P.unfused_causal_attention(q[0], k, k, scale=1.0)
    with pytest.raises(ValueError, match="share shape"):
        P.unfused_causal_attention(q, k, k[:, :, :4], scale=1.0, query_start=0)
    with pytest.raises(ValueError, match="heads must match"):
        P.unfused_causal_attention(q, k[:, :1], k[:, :1], scale=1.0, query_start=0)


# ------------------------------------------------------------------ fused --
def test_fused_entry_points_refuse_cpu_fp32_odd_head_dims_and_dropout():
    q = torch.randn(1, 2, 128, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        P.flash_causal_attention(q, q, q, scale=1.0)
    with pytest.raises(RuntimeError, match="CUDA"):
        P.flash_ring_causal_attention(q, q, q, scale=1.0, cp_group=None, cp_rank=0, cp_size=1, backend=None)
    with pytest.raises(NotImplementedError, match="dropout"):
        P.flash_ring_causal_attention(q, q, q, scale=1.0, cp_group=None, cp_rank=0, cp_size=2, backend=None,
                                      dropout_p=0.1)


# ------------------------------------------------------------------ merge --
@pytest.mark.parametrize("split", [1, 5, 11])
def test_online_softmax_merge_of_two_key_ranges_equals_attention_over_their_union(split):
    torch.manual_seed(1)
    b, h, s, d = 2, 3, 12, 4
    q, k, v = (torch.randn(b, h, s, d) for _ in range(3))

    def partial(ks, vs):
        scores = torch.einsum("bhqd,bhkd->bhqk", q, ks)               # no mask: the merge itself is under test
        lse = torch.logsumexp(scores, dim=-1)                          # [B, h, S]
        out = torch.softmax(scores, dim=-1) @ vs                       # [B, h, S, d]
        return out.transpose(1, 2).contiguous(), lse                   # out as [B, S, h, d]

    out_a, lse_a = partial(k[:, :, :split], v[:, :, :split])
    out_b, lse_b = partial(k[:, :, split:], v[:, :, split:])
    out, lse = AB._online_softmax_combine(out_a, lse_a, out_b, lse_b)
    want_out, want_lse = partial(k, v)
    assert torch.allclose(out, want_out, atol=1e-5) and torch.allclose(lse, want_lse, atol=1e-5)
    # merging is symmetric
    out2, lse2 = AB._online_softmax_combine(out_b, lse_b, out_a, lse_a)
    assert torch.allclose(out2, out, atol=1e-6) and torch.allclose(lse2, lse, atol=1e-6)


@pytest.mark.parametrize("heads_first", [False, True])
def test_partial_attention_merge_accepts_both_output_layouts(heads_first):
    """Two partial attentions over disjoint key sets merged by their log-sum-exps equal
    attention over all keys, for outputs laid out ``[B, S, h, d]`` or ``[B, h, S, d]``."""
    from nano_megatron_b200.parallel.attention_backend import _online_softmax_combine

    torch.manual_seed(0)
    b, h, s, d = 2, 3, 5, 4
    q = torch.randn(b, h, s, d)
    parts, scores = [], []
    for n_keys in (6, 7):
        k, v = torch.randn(b, h, n_keys, d), torch.randn(b, h, n_keys, d)
        sc = q @ k.transpose(-2, -1) * d ** -0.5
        scores.append(sc)
        parts.append((torch.softmax(sc, -1) @ v, torch.logsumexp(sc, -1), v))
    full = torch.cat(scores, -1)
    want = torch.softmax(full, -1) @ torch.cat([p[2] for p in parts], 2)
    lay = (lambda t: t) if heads_first else (lambda t: t.transpose(1, 2).contiguous())
    out, lse = _online_softmax_combine(lay(parts[0][0]), parts[0][1], lay(parts[1][0]), parts[1][1])
    torch.testing.assert_close(out, lay(want), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(lse, torch.logsumexp(full, -1), atol=1e-5, rtol=1e-5)
    with pytest.raises(ValueError):
        _online_softmax_combine(parts[0][0], parts[0][1], parts[1][0][:, :, :2], parts[1][1])

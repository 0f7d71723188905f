"""Pipeline point-to-point helpers against a recording backend (no process
group): which calls are made at the ends and in the middle of a pipeline, with
which peers and buffers, and how deferred sends are drained."""
from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

from nano_megatron_b200.parallel.config import ParallelConfig
from nano_megatron_b200.schedules import p2p


class _Recorder:
    def __init__(self, with_isend: bool):
        self.log = []
        if with_isend:
            self.isend = self._isend

    def send(self, tensor, *, dst, group=None):
        self.log.append(("send", dst, tuple(tensor.shape), group))

    def recv(self, tensor, *, src, group=None):
        self.log.append(("recv", src, tuple(tensor.shape), group))
        tensor.fill_(float(src))
        return tensor

    def _isend(self, tensor, *, dst, group=None):
        self.log.append(("isend", dst, tuple(tensor.shape), group))
        log = self.log

        class _Work:
            def wait(self_inner):
                log.append(("wait", dst))

        return _Work()


def _ctx(pp_rank: int, pp_size: int, backend, *, tp: int = 1, order: str = "tp-cp-dp-pp"):
    cfg = ParallelConfig(tensor_parallel_size=tp, pipeline_parallel_size=pp_size, order=order)
    return SimpleNamespace(
        config=cfg, backend=backend, pipeline_parallel_group="PP",
        pipeline_parallel_rank=pp_rank, pipeline_parallel_size=pp_size,
        tensor_parallel_rank=0, tensor_parallel_size=tp, context_parallel_rank=0, context_parallel_size=1,
        data_parallel_rank=0, data_parallel_size=1)


@pytest.fixture(autouse=True)
def _no_leftover_sends():
    p2p._PENDING_SENDS.clear()
    yield
    p2p._PENDING_SENDS.clear()


def test_first_stage_has_no_upstream_and_last_stage_no_downstream():
    be = _Recorder(with_isend=False)
    first, last = _ctx(0, 3, be), _ctx(2, 3, be)
    kw = dict(shape=(2, 3), dtype=torch.float32, device=torch.device("cpu"))
    assert p2p.recv_forward(first, **kw) is None
    assert p2p.recv_backward(last, **kw) is None
    p2p.send_backward(first, torch.zeros(2, 3))
    p2p.send_forward(last, torch.zeros(2, 3))
    assert be.log == []


def test_single_stage_pipeline_is_all_noops():
    be = _Recorder(with_isend=True)
    only = _ctx(0, 1, be)
    kw = dict(shape=(1,), dtype=torch.float32, device=torch.device("cpu"))
    assert p2p.recv_forward(only, **kw) is None and p2p.recv_backward(only, **kw) is None
    p2p.send_forward(only, torch.zeros(1))
    p2p.send_backward(only, torch.zeros(1))
    assert be.log == [] and p2p._PENDING_SENDS == []


def test_middle_stage_talks_to_both_neighbours_with_blocking_transport():
    be = _Recorder(with_isend=False)
    mid = _ctx(1, 3, be)
    got = p2p.recv_forward(mid, shape=(2, 4), dtype=torch.bfloat16, device=torch.device("cpu"))
    assert got.shape == (2, 4) and got.dtype == torch.bfloat16 and float(got[0, 0]) == 0.0     # from global rank 0
    grad = p2p.recv_backward(mid, shape=(2, 4), dtype=torch.float32, device=torch.device("cpu"))
    assert float(grad[0, 0]) == 2.0                                                             # from global rank 2
    p2p.send_forward(mid, torch.zeros(5))
    p2p.send_backward(mid, torch.zeros(6))
    assert be.log == [("recv", 0, (2, 4), "PP"), ("recv", 2, (2, 4), "PP"), ("send", 2, (5,), "PP"),
                      ("send", 0, (6,), "PP")]
    assert p2p._PENDING_SENDS == []


def test_neighbour_ranks_account_for_tensor_parallel_width_and_order():
    be = _Recorder(with_isend=False)
    # tp = 2, pp = 2, default order: stages are 2 global ranks apart
    p2p.send_forward(_ctx(0, 2, be, tp=2), torch.zeros(1))
    assert be.log[-1][:2] == ("send", 2)
    # pipeline dimension fastest: neighbours are adjacent global ranks
    p2p.send_forward(_ctx(0, 2, be, tp=2, order="pp-tp-cp-dp"), torch.zeros(1))
    assert be.log[-1][:2] == ("send", 1)


def test_deferred_sends_keep_their_tensor_alive_until_drained_in_order():
    be = _Recorder(with_isend=True)
    mid = _ctx(1, 3, be)
    a, b = torch.zeros(2), torch.zeros(3)
    p2p.send_forward(mid, a)
    p2p.send_backward(mid, b)
    assert [e[0] for e in be.log] == ["isend", "isend"]
    assert [t.data_ptr() for _w, t in p2p._PENDING_SENDS] == [a.data_ptr(), b.data_ptr()]
    p2p.drain_pending_sends()
    assert be.log[2:] == [("wait", 2), ("wait", 0)] and p2p._PENDING_SENDS == []
    p2p.drain_pending_sends()                                # idempotent
    assert len(be.log) == 4

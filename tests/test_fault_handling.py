"""Failure detection without touching a GPU: faults are made on the host.

* a rank that leaves between steps -> the survivor's next collective ends with
  an error from the short process-group timeout (Gloo ranks on CPU);
* a message that a test backend drops -> the receiver's bounded wait raises
  ``CommTimeout``;
* a peer that stops sending heartbeats is reported before the next launch
  (``tests/test_aux.py``).
The device-side bounded wait is exercised on a GPU by withholding a flag
(``test_bounded_device_wait_times_out``): the kernel returns a status code and
the context stays usable.
"""
from __future__ import annotations

import os
import sys
import time

import pytest
import torch

from nano_megatron_b200.utils import CommTimeout, StepWatchdog
from tests._dist_utils import launch

HERE = os.path.abspath(__file__)


def worker_rank_leaves_between_steps():
    import datetime
    import torch.distributed as dist
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)                                        # step 1 completes everywhere
    assert t[0].item() == dist.get_world_size()
    if dist.get_rank() == 1:
        os._exit(0)                                           # leaves between steps, nothing in flight
    t0 = time.monotonic()
    try:
        dist.all_reduce(t)
        outcome = "no-error"
    except Exception:
        outcome = "error"
    waited = time.monotonic() - t0
    assert outcome == "error" and waited < 30, (outcome, waited)
    print("PERF survivor saw an error after %.1f s" % waited, flush=True)
    os._exit(0)


def test_survivor_gets_an_error_not_a_hang():
    launch(HERE, "worker_rank_leaves_between_steps", 2, timeout=120)


class _LossyBackend:
    """In-process two-endpoint backend whose ``send`` can drop messages."""

    def __init__(self, drop_every: int = 0):
        self.queue: list[torch.Tensor] = []
        self.sent = 0
        self.drop_every = drop_every

    def send(self, tensor, dst, *, group=None):
        self.sent += 1
        if self.drop_every and self.sent % self.drop_every == 0:
            return                                            # the message is lost
        self.queue.append(tensor.clone())

    def recv(self, tensor, src, *, group=None, deadline_s: float = 0.05):
        StepWatchdog(deadline_s).wait_until(lambda: bool(self.queue), what=f"message from rank {src}")
        tensor.copy_(self.queue.pop(0))
        return tensor


def test_dropped_message_raises_comm_timeout():
    be = _LossyBackend(drop_every=2)
    buf = torch.zeros(3)
    be.send(torch.ones(3), 1)
    assert torch.equal(be.recv(buf, 0), torch.ones(3))
    be.send(torch.full((3,), 2.0), 1)                         # dropped
    with pytest.raises(CommTimeout, match="message from rank 0"):
        be.recv(buf, 0)


def test_raising_rank_is_reported_by_the_launcher():
    with pytest.raises(AssertionError, match="worker_raises"):
        launch(HERE, "worker_raises", 2, timeout=120)


def worker_raises():
    import torch.distributed as dist
    dist.init_process_group("gloo")
    if dist.get_rank() == 1:
        raise RuntimeError("injected host-side failure")
    time.sleep(1.0)


@pytest.mark.gpu
def test_bounded_device_wait_times_out():
    """A flag that nobody sets: the kernel gives up after its budget, stores the
    time-out code and returns; the context keeps working."""
    import ctypes
    from nano_megatron_b200.ops import native

    lib = native.lib()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = native.status_word(flag.device)
    status.zero_()
    budget = 200_000_000                                      # ~0.1 s
    t0 = time.monotonic()
    rc = lib.nmb_bounded_wait_probe(native.ptr(flag), ctypes.c_uint(1), native.ptr(status),
                                    ctypes.c_longlong(budget), native.stream_ptr(flag.device))
    assert rc == 0
    torch.cuda.synchronize()
    assert time.monotonic() - t0 < 5.0
    with pytest.raises(native.NativeKernelError, match="peer flag wait timed out"):
        native.check_status()
    native.check_status()                                     # cleared
    flag.fill_(1)                                             # with the flag set the wait returns at once
    lib.nmb_bounded_wait_probe(native.ptr(flag), ctypes.c_uint(1), native.ptr(status), ctypes.c_longlong(budget),
                               native.stream_ptr(flag.device))
    torch.cuda.synchronize()
    native.check_status()
    assert (torch.ones(4, device="cuda") * 2).sum().item() == 8.0


if __name__ == "__main__":
    from tests._dist_utils import run_worker_if_requested
    run_worker_if_requested(globals())

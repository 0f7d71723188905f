"""Failure detection on the host: step deadlines and rank heartbeats.

The reference has none (a dead peer hangs the job; only its test launchers have
subprocess timeouts, tests/distributed/test_pp_gloo.py:55).  Three pieces:

* :class:`StepWatchdog` -- deadline on the completion of a step (CUDA event
  query or a host flag); raises :class:`CommTimeout` instead of waiting forever.
* :class:`Heartbeat` -- every rank bumps a counter in the rendezvous store
  between steps; peers that stop bumping are reported *before* the next
  collective is launched, so no kernel ever waits on a dead rank.
* process-group timeouts (``parallel.context.DEFAULT_TIMEOUT_S``) end a
  collective whose peer never arrives with an error.

Device-side waits are bounded separately (``csrc/common.cuh``, ``csrc/comm.cu``)
and report through the status word read by :func:`ops.native.check_status`.
Nothing here ever faults, traps or hangs a GPU to provoke a failure.
"""
from __future__ import annotations

import time
from typing import Any, Callable, Optional

import torch


class CommTimeout(RuntimeError):
    """A step, a collective or a peer did not make progress within its deadline."""


class StepWatchdog:
    def __init__(self, deadline_s: float, *, poll_s: float = 0.001) -> None:
        self.deadline_s, self.poll_s = float(deadline_s), float(poll_s)

    def wait_event(self, event: "torch.cuda.Event", what: str = "step") -> float:
        """Poll a recorded CUDA event; returns the seconds waited."""
        t0 = time.monotonic()
        while not event.query():
            if time.monotonic() - t0 > self.deadline_s:
                raise CommTimeout(f"{what} did not finish within {self.deadline_s:.1f} s")
            time.sleep(self.poll_s)
        return time.monotonic() - t0

    def wait_until(self, done: Callable[[], bool], what: str = "condition") -> float:
        t0 = time.monotonic()
        while not done():
            if time.monotonic() - t0 > self.deadline_s:
                raise CommTimeout(f"{what} not reached within {self.deadline_s:.1f} s")
            time.sleep(self.poll_s)
        return time.monotonic() - t0


class Heartbeat:
    """Per-rank liveness counters in a key-value store (``torch.distributed`` store
    or anything with ``set`` / ``get``)."""

    def __init__(self, store: Any, rank: int, world_size: int, *, prefix: str = "nmb_hb") -> None:
        self.store, self.rank, self.world = store, rank, world_size
        self.prefix = prefix
        self._beat = 0
        self._seen: dict[int, tuple[int, float]] = {}

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self) -> None:
        self._beat += 1
        self.store.set(self._key(self.rank), str(self._beat))

    def _read(self, rank: int) -> int:
        try:
            return int(bytes(self.store.get(self._key(rank))).decode())
        except Exception:
            return 0

    def stale_ranks(self, max_age_s: float) -> list[int]:
        """Ranks whose counter has not moved for ``max_age_s`` seconds."""
        now = time.monotonic()
        stale = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            last = self._seen.get(r)
            if last is None or v != last[0]:
                self._seen[r] = (v, now)
            elif now - last[1] > max_age_s:
                stale.append(r)
        return stale

    def check(self, max_age_s: float) -> None:
        stale = self.stale_ranks(max_age_s)
        if stale:
            raise CommTimeout(f"rank(s) {stale} sent no heartbeat for {max_age_s:.1f} s")

"""Randomised-interleaving model of the buffer-reuse protocol of the fused GEMM ->
reduce-scatter / all-reduce launches (``FusedComm`` in ``csrc/gemm_tcgen05.cu``).

The kernels themselves only run on GPUs; what can be checked without one is the
protocol: peers store partial tiles into a rank's staging buffer, that rank reads them,
and a later launch may reuse the buffer.  The rules modelled here are the ones the kernel
implements:

* a launch with epoch ``e`` first publishes "rank r has started e" into every peer's
  memory (``rs_started``);
* every buffer remembers the epoch of the last launch that used it (``rs_last``; the same
  on all ranks because they run the same sequence);
* before its first store into a peer's buffer a rank waits until that peer has started a
  launch LATER than the buffer's last use (launches of a rank are serialised on its
  stream, so "started a later one" means "finished with the earlier one");
* a rank finishes a launch when the partial tiles of all peers for that launch have arrived.

Each rank is a generator that yields at every access to memory another rank can see; a
scheduler picks the next rank at random.  The invariant: nobody stores into a buffer whose
owner has not finished reading it for an earlier launch.  The model shows the three facts
the comments in the kernel claim: with two alternating buffers the wait never blocks and
is not even needed, with a single buffer and no wait the race exists, and with a single
buffer the wait removes it.

The one-launch cross-entropy exchange (``ce_forward_fused_kernel``: every rank stores its
per-token statistics into all ranks' gather buffer chosen by the parity of a device epoch,
then the ranks exchange one flag each and read) is the "two buffers, no wait" case of the
same model.
"""
from __future__ import annotations

import random

import pytest


class _World:
    def __init__(self, n_ranks: int, n_buffers: int, use_wait: bool) -> None:
        self.n, self.nb, self.use_wait = n_ranks, n_buffers, use_wait
        # rank-local memory that peers write: started[r][p] = last epoch rank p announced to r
        self.started = [[0] * n_ranks for _ in range(n_ranks)]
        # staging[r][b][p] = epoch of the partial tile rank p stored for owner r in buffer b
        self.staging = [[[0] * n_ranks for _ in range(n_buffers)] for _ in range(n_ranks)]
        # reading[r][b] = epoch owner r is currently consuming from buffer b (0: none)
        self.reading = [[0] * n_buffers for _ in range(n_ranks)]
        # last_use[r][b]: rank r's own record of the last launch that used buffer b (every rank
        # keeps one; they agree because launches of a rank are serialised and the sequences match)
        self.last_use = [[0] * n_buffers for _ in range(n_ranks)]
        self.blocked_waits = 0
        self.violations: list[str] = []


def _rank(world: _World, r: int, launches: int):
    n = world.n
    for e in range(1, launches + 1):
        b = (e - 1) % world.nb
        need = world.last_use[r][b] + 1 if world.last_use[r][b] else 0
        # 1. announce the start of launch e to every peer
        for p in range(n):
            if p != r:
                world.started[p][r] = e
                yield
        # 2. partial tiles for the other owners
        for o in range(n):
            if o == r:
                continue
            if world.use_wait:
                while world.started[r][o] < need:
                    world.blocked_waits += 1
                    yield
            busy = world.reading[o][b]
            if busy and busy < e:
                world.violations.append(f"rank {r} stored launch {e} into buffer {b} of rank {o} "
                                        f"while it was still reading launch {busy}")
            world.staging[o][b][r] = e
            yield
        # 3. own tiles: wait for the peers' partials of THIS launch, then read them
        for p in range(n):
            if p != r:
                while world.staging[r][b][p] < e:
                    yield
        world.reading[r][b] = e
        for p in range(n):
            if p != r:
                if world.staging[r][b][p] != e:
                    world.violations.append(f"rank {r} read launch {world.staging[r][b][p]} data in launch {e}")
                yield
        world.reading[r][b] = 0
        # 4. what the stream does with the result afterwards still belongs to launch e
        yield
        world.last_use[r][b] = e
        yield


def _run(n_ranks: int, n_buffers: int, use_wait: bool, launches: int, seed: int) -> _World:
    rng = random.Random(seed)
    world = _World(n_ranks, n_buffers, use_wait)
    ranks = {r: _rank(world, r, launches) for r in range(n_ranks)}
    steps = 0
    while ranks:
        r = rng.choice(list(ranks))
        try:
            next(ranks[r])
        except StopIteration:
            del ranks[r]
        steps += 1
        assert steps < 2_000_000, "the model dead-locked"
    return world


@pytest.mark.parametrize("n_ranks", [2, 4, 8])
def test_two_alternating_buffers_need_no_wait_and_the_wait_never_blocks(n_ranks):
    for seed in range(40):
        free = _run(n_ranks, 2, False, launches=12, seed=seed)
        assert not free.violations, free.violations[:3]
        guarded = _run(n_ranks, 2, True, launches=12, seed=seed)
        assert not guarded.violations and guarded.blocked_waits == 0


@pytest.mark.parametrize("n_ranks", [2, 4])
def test_a_single_buffer_races_without_the_wait_and_not_with_it(n_ranks):
    raced = 0
    for seed in range(60):
        if _run(n_ranks, 1, False, launches=12, seed=seed).violations:
            raced += 1
        guarded = _run(n_ranks, 1, True, launches=12, seed=seed)
        assert not guarded.violations, guarded.violations[:3]
    assert raced > 0, "the model never produced the race the wait is there for"

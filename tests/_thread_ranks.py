"""In-process multi-rank simulator for the CommBackend protocol.

``run_ranks(n, fn)`` runs ``fn(rank, backend)`` on ``n`` threads; the backend
objects share one rendezvous, so collectives exchange real data between the
"ranks".  CPU autograd runs a backward pass on the thread that called it, so
whole forward + backward passes of the parallel operators can be checked for
exact arithmetic without processes or sockets.  (The socket-based Gloo tests
cover the real transport; this covers the maths, quickly and for any rank
count.)
"""
from __future__ import annotations

import threading
from typing import Any, Callable, Optional

import torch
from torch import Tensor

_OPS = {
    "sum": lambda ts: torch.stack(ts).sum(0),
    "max": lambda ts: torch.stack(ts).max(0).values,
    "min": lambda ts: torch.stack(ts).min(0).values,
    "product": lambda ts: torch.stack(ts).prod(0),
}


class _Meeting:
    """Exchange point of one group of ranks."""

    def __init__(self, members: tuple[int, ...]) -> None:
        self.members = members
        self.barrier = threading.Barrier(len(members), timeout=30)
        self.slots: list[Any] = [None] * len(members)

    def exchange(self, rank: int, item: Any) -> list[Any]:
        """Every member deposits one item and gets all members' items (member order)."""
        self.slots[self.members.index(rank)] = item
        self.barrier.wait()
        items = list(self.slots)
        self.barrier.wait()            # nobody overwrites a slot that is still being read
        return items


class _Rendezvous:
    def __init__(self, n: int) -> None:
        self.n = n
        self._lock = threading.Lock()
        self._meetings: dict[tuple[int, ...], _Meeting] = {}
        self.mail: dict[tuple[int, int], list[Tensor]] = {}
        self.mail_cv = threading.Condition()
        self.barrier = self.meeting(None).barrier

    def meeting(self, group: Any) -> _Meeting:
        members = tuple(range(self.n)) if group is None else tuple(group)
        with self._lock:
            if members not in self._meetings:
                self._meetings[members] = _Meeting(members)
            return self._meetings[members]

    def exchange(self, rank: int, item: Any, group: Any = None) -> list[Any]:
        return self.meeting(group).exchange(rank, item)

    def abort(self) -> None:
        with self._lock:
            for m in self._meetings.values():
                m.barrier.abort()


class _Done:
    def wait(self) -> None:
        return None


class ThreadBackend:
    """One per simulated rank.  A ``group`` is ``None`` (all ranks) or a tuple of
    global ranks; a rank's position in the tuple is its rank in the group."""

    def __init__(self, rank: int, rdv: _Rendezvous) -> None:
        self.rank, self._rdv = rank, rdv
        self.counts: dict[str, int] = {}

    def _count(self, name: str) -> None:
        self.counts[name] = self.counts.get(name, 0) + 1

    def all_reduce(self, tensor: Tensor, *, group: Optional[Any] = None, op: str = "sum", async_op: bool = False):
        self._count("all_reduce")
        parts = self._rdv.exchange(self.rank, tensor.detach().clone(), group)
        tensor.copy_(_OPS[op](parts))
        return _Done() if async_op else tensor

    def reduce_scatter(self, output: Tensor, input_list: list[Tensor], *, group: Optional[Any] = None,
                       op: str = "sum") -> Tensor:
        self._count("reduce_scatter")
        everyone = self._rdv.exchange(self.rank, [t.detach().clone() for t in input_list], group)
        me = self.rank if group is None else tuple(group).index(self.rank)
        output.copy_(_OPS[op]([lst[me] for lst in everyone]))
        return output

    def all_gather(self, tensor_list: list[Tensor], tensor: Tensor, *, group: Optional[Any] = None) -> list[Tensor]:
        self._count("all_gather")
        for dst, src in zip(tensor_list, self._rdv.exchange(self.rank, tensor.detach().clone(), group)):
            dst.copy_(src)
        return tensor_list

    def all_gather_into_tensor(self, output: Tensor, input: Tensor, *, group: Optional[Any] = None) -> Tensor:
        self._count("all_gather_into_tensor")
        parts = self._rdv.exchange(self.rank, input.detach().clone(), group)
        if output.dim() == input.dim():
            output.copy_(torch.cat(parts, dim=0))
        else:
            output.copy_(torch.stack(parts, dim=0))
        return output

    def broadcast(self, tensor: Tensor, src: int, *, group: Optional[Any] = None) -> Tensor:
        self._count("broadcast")
        members = tuple(range(self._rdv.n)) if group is None else tuple(group)
        tensor.copy_(self._rdv.exchange(self.rank, tensor.detach().clone(), group)[members.index(src)])   # src is global
        return tensor

    def send(self, tensor: Tensor, dst: int, *, group: Optional[Any] = None) -> None:
        self._count("send")
        with self._rdv.mail_cv:
            self._rdv.mail.setdefault((self.rank, dst), []).append(tensor.detach().clone())
            self._rdv.mail_cv.notify_all()

    def recv(self, tensor: Tensor, src: int, *, group: Optional[Any] = None) -> Tensor:
        self._count("recv")
        key = (src, self.rank)
        with self._rdv.mail_cv:
            ok = self._rdv.mail_cv.wait_for(lambda: self._rdv.mail.get(key), timeout=30)
            if not ok:
                raise TimeoutError(f"rank {self.rank}: nothing arrived from rank {src}")
            tensor.copy_(self._rdv.mail[key].pop(0))
        return tensor

    def barrier(self, *, group: Optional[Any] = None) -> None:
        self._rdv.exchange(self.rank, None, group)


def run_ranks(n: int, fn: Callable[..., Any], prepare: Optional[Callable[[int, ThreadBackend], Any]] = None) -> list[Any]:
    """Run ``fn(rank, backend)`` for ``n`` simulated ranks; returns their results
    in rank order and re-raises the first failure.  With ``prepare``, the main
    thread first calls ``prepare(rank, backend)`` for every rank in turn (the
    place to build modules: the global random generator is shared between
    threads) and the ranks run ``fn(rank, backend, prepared)``."""
    rdv = _Rendezvous(n)
    backends = [ThreadBackend(r, rdv) for r in range(n)]
    prepared = [prepare(r, backends[r]) for r in range(n)] if prepare is not None else None
    results: list[Any] = [None] * n
    errors: list[Optional[BaseException]] = [None] * n

    def body(rank: int) -> None:
        try:
            if prepared is not None:
                results[rank] = fn(rank, backends[rank], prepared[rank])
            else:
                results[rank] = fn(rank, backends[rank])
        except BaseException as exc:  # noqa: BLE001 - reported to the caller below
            errors[rank] = exc
            rdv.abort()

    threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    real = [e for e in errors if e is not None and not isinstance(e, threading.BrokenBarrierError)]
    if real:
        raise real[0]
    if any(e is not None for e in errors):
        raise errors[[i for i, e in enumerate(errors) if e is not None][0]]
    if any(t.is_alive() for t in threads):
        raise TimeoutError("a simulated rank did not finish")
    return results


def thread_context(rank: int, backend: ThreadBackend, *, tp: int = 1, pp: int = 1, cp: int = 1, dp: int = 1,
                   sequence_parallel: bool = False, order: str = "tp-cp-dp-pp"):
    """A ``ParallelContext`` for simulated rank ``rank`` whose groups are tuples of
    global ranks (what :class:`ThreadBackend` understands)."""
    from nano_megatron_b200.parallel.config import ParallelConfig
    from nano_megatron_b200.parallel.context import ParallelContext
    from nano_megatron_b200.parallel.rank_generator import RankGenerator

    gen = RankGenerator(tp=tp, dp=dp, pp=pp, cp=cp, order=order)
    coords = gen.decode(rank)

    def group_of(token: str):
        for g in gen.get_ranks(token):
            if rank in g:
                return tuple(g)
        raise AssertionError(token)

    cfg = ParallelConfig(tensor_parallel_size=tp, pipeline_parallel_size=pp, context_parallel_size=cp,
                         data_parallel_size=dp, sequence_parallel=sequence_parallel, order=order)
    return ParallelContext(
        config=cfg, rank=rank, world_size=gen.world_size, local_rank=rank, backend=backend,
        tensor_parallel_size=tp, tensor_parallel_rank=coords["tp"], data_parallel_size=dp,
        data_parallel_rank=coords["dp"], pipeline_parallel_size=pp, pipeline_parallel_rank=coords["pp"],
        context_parallel_size=cp, context_parallel_rank=coords["cp"], tensor_parallel_group=group_of("tp"),
        data_parallel_group=group_of("dp"), pipeline_parallel_group=group_of("pp"),
        context_parallel_group=group_of("cp"), sequence_parallel=sequence_parallel,
        data_context_parallel_group=group_of("dp-cp"))

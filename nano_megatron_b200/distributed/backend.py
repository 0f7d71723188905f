"""Communication backend protocol.

Model, DDP and schedule code move data only through an object with these eight
methods (nano_megatron/distributed/backend.py:8-47 in the reference), so a
backend can be swapped at ``initialize_parallel(backend=...)``.  Reduce ops are
the strings ``"sum" | "max" | "min" | "product"``.
"""
from __future__ import annotations

from typing import Any, Optional, Protocol, runtime_checkable

from torch import Tensor


@runtime_checkable
class CommBackend(Protocol):
    def all_reduce(self, tensor: Tensor, *, group: Optional[Any] = None, op: str = "sum",
                   async_op: bool = False) -> Any: ...

    def reduce_scatter(self, output: Tensor, input_list: list[Tensor], *, group: Optional[Any] = None,
                       op: str = "sum") -> Tensor: ...

    def all_gather(self, tensor_list: list[Tensor], tensor: Tensor, *,
                   group: Optional[Any] = None) -> list[Tensor]: ...

    def all_gather_into_tensor(self, output: Tensor, input: Tensor, *,
                               group: Optional[Any] = None) -> Tensor: ...

    def send(self, tensor: Tensor, dst: int, *, group: Optional[Any] = None) -> None: ...

    def recv(self, tensor: Tensor, src: int, *, group: Optional[Any] = None) -> Tensor: ...

    def broadcast(self, tensor: Tensor, src: int, *, group: Optional[Any] = None) -> Tensor: ...

    def barrier(self, *, group: Optional[Any] = None) -> None: ...

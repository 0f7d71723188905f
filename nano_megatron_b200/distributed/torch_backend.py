"""``CommBackend`` on ``torch.distributed`` (NCCL on GPUs, Gloo on CPU);
the counterpart of nano_megatron/distributed/torch_backend.py:8-80."""
from __future__ import annotations

from typing import Any, Optional

import torch.distributed as dist
from torch import Tensor

_REDUCE_OPS = {
    "sum": dist.ReduceOp.SUM,
    "max": dist.ReduceOp.MAX,
    "min": dist.ReduceOp.MIN,
    "product": dist.ReduceOp.PRODUCT,
}


def reduce_op_from_string(op: str) -> dist.ReduceOp:
    try:
        return _REDUCE_OPS[op.lower()]
    except KeyError:
        raise ValueError(f"unsupported reduce op: {op!r}") from None


def _refuse_inside_capture(tensor: Tensor) -> None:
    """The step engines capture a step into a CUDA graph only when every
    collective in it is a peer-memory kernel of this package.  A shape that
    falls back to a library collective during the capture would put an NCCL
    kernel into the graph; refuse instead, so the engine stays eager."""
    if tensor.is_cuda:
        import torch
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("library collective requested inside a CUDA graph capture")


class TorchDistBackend:
    """Thin, stateless wrapper; ``all_reduce`` is the only op with an async mode."""

    def all_reduce(self, tensor: Tensor, *, group: Optional[Any] = None, op: str = "sum",
                   async_op: bool = False) -> Any:
        _refuse_inside_capture(tensor)
        work = dist.all_reduce(tensor, op=reduce_op_from_string(op), group=group, async_op=async_op)
        return work if async_op else tensor

    def reduce_scatter(self, output: Tensor, input_list: list[Tensor], *, group: Optional[Any] = None,
                       op: str = "sum") -> Tensor:
        _refuse_inside_capture(output)
        dist.reduce_scatter(output, input_list, op=reduce_op_from_string(op), group=group)
        return output

    def all_gather(self, tensor_list: list[Tensor], tensor: Tensor, *,
                   group: Optional[Any] = None) -> list[Tensor]:
        _refuse_inside_capture(tensor)
        dist.all_gather(tensor_list, tensor, group=group)
        return tensor_list

    def all_gather_into_tensor(self, output: Tensor, input: Tensor, *,
                               group: Optional[Any] = None) -> Tensor:
        _refuse_inside_capture(output)
        dist.all_gather_into_tensor(output, input, group=group)
        return output

    def send(self, tensor: Tensor, dst: int, *, group: Optional[Any] = None) -> None:
        dist.send(tensor, dst, group=group)

    def recv(self, tensor: Tensor, src: int, *, group: Optional[Any] = None) -> Tensor:
        dist.recv(tensor, src, group=group)
        return tensor

    def broadcast(self, tensor: Tensor, src: int, *, group: Optional[Any] = None) -> Tensor:
        _refuse_inside_capture(tensor)
        dist.broadcast(tensor, src=src, group=group)
        return tensor

    def barrier(self, *, group: Optional[Any] = None) -> None:
        dist.barrier(group=group)

    # Extras beyond the eight-method protocol: non-blocking point-to-point, used
    # by the pipeline schedule so a send does not stall the compute stream.
    def isend(self, tensor: Tensor, dst: int, *, group: Optional[Any] = None) -> Any:
        return dist.isend(tensor, dst, group=group)

    def irecv(self, tensor: Tensor, src: int, *, group: Optional[Any] = None) -> Any:
        return dist.irecv(tensor, src, group=group)

"""Pipeline schedules and their point-to-point helpers."""
from .one_f_one_b import forward_backward_1f1b, warmup_microbatches
from .p2p import recv_backward, recv_forward, send_backward, send_forward

__all__ = ["forward_backward_1f1b", "recv_backward", "recv_forward", "send_backward", "send_forward",
           "warmup_microbatches"]

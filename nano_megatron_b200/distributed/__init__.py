"""Communication backend abstraction, gradient buckets and the data-parallel wrapper."""
from .backend import CommBackend
from .bucket import GradBucket, build_buckets
from .ddp import DistributedDataParallel
from .symm_backend import SymmetricBackend
from .torch_backend import TorchDistBackend, reduce_op_from_string

__all__ = ["CommBackend", "DistributedDataParallel", "GradBucket", "SymmetricBackend", "TorchDistBackend",
           "build_buckets", "reduce_op_from_string"]

"""Distributed training: process group, collectives, symmetric heap, DDP.
Parity: reference `genesis/distributed/__init__.py` import surface."""
from .process_group import (init_process_group, destroy_process_group, get_world_size, get_rank,
                            get_local_rank, get_backend, is_initialized, CommTimeout)
from .collectives import (ReduceOp, all_reduce, all_gather, broadcast, reduce_scatter, all_to_all_single,
                          barrier)
from . import symm
from . import watchdog
from .watchdog import Heartbeat
from . import comm, nccl_backend  # noqa: F401  (module paths of the reference)


def __getattr__(name):
    if name in ("DistributedDataParallel", "DDP"):
        from ..nn.parallel import DistributedDataParallel
        return DistributedDataParallel
    if name == "parallel":
        from . import parallel
        return parallel
    raise AttributeError(name)

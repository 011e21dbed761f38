"""Process-group lifecycle. Parity: reference `genesis/distributed/process_group.py:26-127`
(API, env handling `WORLD_SIZE/RANK/LOCAL_RANK`, error strings).

Plumbing is `torch.distributed`: backend "nccl" means "GPU collectives" (NCCL communicator
for cold paths and A/B runs, plus the peer-memory kernels of `genesis_b200.distributed.symm`
for the hot paths); "gloo" runs the same host-side logic on CPU ranks, which is what the
multi-process CPU tests use.  With `world_size == 1` no communicator is created and every
collective is a no-op, as in the reference (`nccl_backend.py:61-66`).  Rendezvous goes through
`init_method` (default `tcp://127.0.0.1:23456`, or the `MASTER_ADDR/MASTER_PORT` a launcher set).
"""
import datetime
import logging
import os

import torch
import torch.distributed as tdist

logger = logging.getLogger(__name__)

_world_size = None
_rank = None
_local_rank = None
_initialized = False
_backend = None
_owns_torch_pg = False


class CommTimeout(RuntimeError):
    """A collective (host- or device-side wait) ran out of its time budget."""


def init_process_group(backend="nccl", init_method=None, world_size=None, rank=None, timeout_s=None):
    global _world_size, _rank, _local_rank, _initialized, _backend, _owns_torch_pg
    if _initialized:
        return
    b = backend.lower()
    if b == "mpi":
        raise NotImplementedError("MPI backend not implemented yet")
    if b not in ("nccl", "gloo"):
        raise ValueError(f"Unsupported backend: {backend}")
    if world_size is None:
        world_size = int(os.environ.get("WORLD_SIZE", 1))
    if rank is None:
        rank = int(os.environ.get("RANK", 0))
    _local_rank = int(os.environ.get("LOCAL_RANK", rank if b == "nccl" else 0))
    if world_size > 1:
        if b == "nccl":
            if not torch.cuda.is_available():
                raise RuntimeError("NCCL library not available: CUDA is not available on this machine")
            torch.cuda.set_device(_local_rank % torch.cuda.device_count())
        if not tdist.is_initialized():
            if init_method is None:
                if "MASTER_ADDR" in os.environ and "MASTER_PORT" in os.environ:
                    init_method = "env://"
                else:
                    init_method = "tcp://127.0.0.1:23456"
            init_method = init_method.replace("tcp://localhost", "tcp://127.0.0.1")
            timeout = datetime.timedelta(seconds=float(
                timeout_s if timeout_s is not None else os.environ.get("GENESIS_COMM_TIMEOUT_S", 600)))
            kw = {}
            if b == "nccl":
                kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
            tdist.init_process_group(backend=b, init_method=init_method, world_size=world_size, rank=rank,
                                     timeout=timeout, **kw)
            _owns_torch_pg = True
    _world_size, _rank, _backend = world_size, rank, b
    _initialized = True
    logger.info("Initialized distributed process group: rank=%d, world_size=%d, local_rank=%d",
                rank, world_size, _local_rank)


def destroy_process_group():
    """Idempotent teardown: frees peer mappings, then the communicator."""
    global _world_size, _rank, _local_rank, _initialized, _backend, _owns_torch_pg
    if not _initialized:
        return
    from . import symm
    symm.shutdown()
    if _owns_torch_pg and tdist.is_initialized():
        try:
            tdist.destroy_process_group()
        except Exception as e:  # a dead peer must not block teardown
            logger.warning("destroy_process_group: %s", e)
    _world_size = _rank = _local_rank = _backend = None
    _initialized = False
    _owns_torch_pg = False
    logger.info("Destroyed distributed process group")


def _check():
    if not _initialized:
        raise RuntimeError("Process group not initialized")


def get_world_size():
    _check()
    return _world_size


def get_rank():
    _check()
    return _rank


def get_local_rank():
    _check()
    return _local_rank


def get_backend():
    _check()
    return _backend


def is_initialized():
    return _initialized


def barrier():
    """Block until every rank of the group arrives (reference `distributed/process_group.py:118-127`)."""
    _check()
    from . import collectives
    collectives.barrier()

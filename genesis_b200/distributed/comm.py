"""`genesis.distributed.comm` of the reference: the collectives API."""
from .collectives import ReduceOp, all_gather, all_reduce, barrier, broadcast, reduce_scatter  # noqa: F401

"""Parallelism strategies: data parallel (`ddp`) and expert parallel (`ep`)."""
from . import ep
from ..nn.parallel import DistributedDataParallel

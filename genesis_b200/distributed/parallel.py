"""`genesis.distributed.parallel` of the reference."""
from ..nn.parallel import DistributedDataParallel  # noqa: F401

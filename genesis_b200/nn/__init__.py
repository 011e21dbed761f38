from . import functional
from .modules import *  # noqa: F401,F403
from .modules import Module, Parameter
from . import utils
from . import parallel
from .parallel import DistributedDataParallel
from . import attention, layer_norm, triton_ops  # noqa: E402,F401  (submodules the reference's `genesis.nn` exposes)

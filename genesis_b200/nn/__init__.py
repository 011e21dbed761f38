from . import functional
from .modules import *  # noqa: F401,F403
from .modules import Module, Parameter
from . import utils
from . import parallel
from .parallel import DistributedDataParallel

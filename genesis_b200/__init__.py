"""genesis_b200: a Blackwell-native deep-learning framework with the capabilities and public
API of Genesis (import surface parity: reference `genesis/__init__.py:9-72`).

    import genesis_b200 as genesis
"""
__version__ = "0.1.0"

from .dtypes import (float32, float16, float64, bfloat16, int32, int64, int16, int8, uint8, bool,  # noqa: A004
                     get_dtype, is_floating_point, is_integer, DType)
from .amp_state import amp_state as _amp_state
from .tensor import Tensor, make_tensor, tensor
from .init import (rand, randn, randn_like, randint, ones, zeros, full, full_like, empty, empty_like, zeros_like,
                   ones_like, one_hot, eye, arange, outer, from_numpy, multinomial)
from .serialization import save, load, save_checkpoint, load_checkpoint
from .grad_mode import no_grad, enable_grad, set_grad_enabled, is_grad_enabled
from . import nn
from . import init
from . import optim
from . import utils
from . import amp
from . import distributed
from . import ops
from .function import Function, AMPPolicy
from .functional import (triu, tril, isinf, isnan, isfinite, argsort, sort, bincount, nonzero, allclose,
                         eq, ne, gt, ge, lt, le)
from . import cuda
from .api import bind_tensor_methods, bind_nn_functional_methods
bind_tensor_methods()
bind_nn_functional_methods()
from .random import (seed, manual_seed, initial_seed, get_rng_state, set_rng_state, default_generator,  # noqa: E402
                     fork_rng, Generator)
from .device import device, Device  # noqa: E402
from .nn.functional import (add, sub, mul, div, pow, neg, exp, log, sqrt, sin, cos, tanh, abs, matmul,  # noqa: E402,A004
                            sum, mean, max, min, maximum, where, cat, stack, reshape, transpose, permute,
                            squeeze, unsqueeze, clamp, topk, softmax, log_softmax, relu, sigmoid, gather,
                            scatter, scatter_add, repeat_interleave, logsumexp, argmax, argmin, var, std, split)
from . import models  # noqa: E402
from . import parallel  # noqa: E402
from . import backends  # noqa: E402
from . import storage  # noqa: E402
from .backends import Storage, CPUStorage, CUDAStorage  # noqa: E402,F401
from .device import DeviceType  # noqa: E402,F401
from .ops.dispatcher import OperationDispatcher  # noqa: E402,F401
Dispatcher = OperationDispatcher      # the name `genesis.functional` gives it in the reference


def _export_functional():
    """The reference star-exports its whole functional namespace at top level (`genesis/__init__.py:52-57`:
    `from .backends import *`, `from .functional import *`, where `functional.py:10` star-imports `nn.functional`):
    every public function and Function class of `nn.functional` is reachable as `genesis.<name>` too."""
    import types
    from .nn import functional as _F
    g = globals()
    for name, obj in vars(_F).items():
        if name.startswith("_") or isinstance(obj, types.ModuleType) or name in g:
            continue
        g[name] = obj


_export_functional()

use_triton = False   # kept for API parity; there is no Triton path


def cuda_available():
    return cuda.is_available()


def __getattr__(name):
    # module-level autocast flags of the reference, backed by thread-local state
    if name == "enable_autocast":
        return _amp_state.enabled
    if name == "amp_dtype":
        return get_dtype(_amp_state.dtype)
    if name == "upgrade":
        return False
    raise AttributeError(f"module 'genesis_b200' has no attribute {name!r}")

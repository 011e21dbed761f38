"""`genesis.nn.triton_ops` import path of the reference (`nn/triton_ops/__init__.py:1-6`).  There is no Triton here:
the names resolve to the sm_100a kernels behind `genesis_b200.nn.functional`, and the submodules of the reference
(`dropout`, `gelu`, `silu`, `softmax`, `layer_norm`, `rmsnorm`, `grad_check`) exist under the same names."""
# submodules first, then the functions: `genesis.nn.triton_ops.softmax` is the function, as in the reference, while
# `from genesis.nn.triton_ops.softmax import safe_softmax` reaches the module
from . import dropout, gelu, grad_check, layer_norm, rmsnorm, silu, softmax  # noqa: F401,E402
from ..functional import (dropout, softmax, safe_softmax, silu, gelu, fused_layer_norm, fused_rmsnorm,  # noqa: F401,F811,E402
                          FusedLayerNormFunction, FusedRMSNormFunction, DropoutFunction)

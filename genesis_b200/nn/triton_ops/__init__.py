"""`genesis.nn.triton_ops` import path of the reference (`nn/triton_ops/__init__.py:1-6`).  There is no Triton here:
the names resolve to the sm_100a kernels behind `genesis_b200.nn.functional`, and the submodules of the reference
(`dropout`, `gelu`, `silu`, `softmax`, `layer_norm`, `rmsnorm`, `grad_check`) exist under the same names."""
from ..functional import (dropout, softmax, safe_softmax, silu, gelu, fused_layer_norm, fused_rmsnorm,  # noqa: F401
                         FusedLayerNormFunction, FusedRMSNormFunction, DropoutFunction)

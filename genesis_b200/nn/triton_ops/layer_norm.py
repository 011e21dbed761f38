"""`genesis.nn.triton_ops.layer_norm` of the reference: fused LayerNorm forward / backward (kernels of `genesis_b200/csrc`)."""
from ...nn.functional import FusedLayerNormFunction, fused_layer_norm  # noqa: F401

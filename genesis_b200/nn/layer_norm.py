"""`genesis.nn.layer_norm` import path of the reference (`nn/layer_norm.py:123-213`)."""
from .functional import FusedLayerNormFunction, fused_layer_norm  # noqa: F401

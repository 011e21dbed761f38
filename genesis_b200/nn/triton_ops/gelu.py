"""`genesis.nn.triton_ops.gelu` of the reference: GELU forward / backward (kernels of `genesis_b200/csrc`)."""
from ...nn.functional import GELUFunction, gelu  # noqa: F401

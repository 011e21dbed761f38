"""`genesis.nn.triton_ops.rmsnorm` of the reference: fused RMSNorm forward / backward (kernels of `genesis_b200/csrc`)."""
from ...nn.functional import FusedRMSNormFunction, fused_rmsnorm  # noqa: F401

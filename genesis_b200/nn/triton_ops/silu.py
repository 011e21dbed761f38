"""`genesis.nn.triton_ops.silu` of the reference: SiLU forward / backward (kernels of `genesis_b200/csrc`)."""
from ...nn.functional import SiLUFunction, silu  # noqa: F401

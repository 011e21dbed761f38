"""`genesis.nn.triton_ops.dropout` of the reference: Philox dropout with its mask kernel (kernels of `genesis_b200/csrc`)."""
from ...nn.functional import DropoutFunction, dropout  # noqa: F401

"""`genesis.optim.adamw` of the reference: `AdamW`, and the fused update under the name of its kernel
(`fused_adamw_kernel` = the multi-tensor update of `csrc/optim.cu`, `ops.dispatch.adamw_step`)."""
from ..ops.dispatch import adamw_step as fused_adamw_kernel  # noqa: F401
from .optimizer import AdamW  # noqa: F401

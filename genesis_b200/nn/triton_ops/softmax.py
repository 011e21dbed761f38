"""`genesis.nn.triton_ops.softmax` of the reference: `softmax`, `safe_softmax` and their Function classes (the tiling
heuristics of its Triton kernels have no counterpart: the CUDA kernels pick warp-per-row, register-resident or streamed
shared-memory variants by row length, `csrc/softmax_ce.cu`)."""
from ...nn.functional import SoftmaxFunction, safe_softmax, softmax  # noqa: F401

SafeSoftmaxFunction = SoftmaxFunction
OnlineSoftmaxFunction = SoftmaxFunction

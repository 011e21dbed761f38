"""CUDA graphs for launch-bound loops: capture a fixed sequence of the framework's kernels once, replay it with one
launch.

The native kernels are launched on torch's current stream with plain runtime launches, and temporaries come from
torch's (or the native pool's) stream-ordered allocator, so a region that does no host read (`.item()`, `.numpy()`,
`check_status`) and changes no launch arguments between replays is capturable as is.  Rules of use:

* run the region eagerly a few times first (`warmup`): kernels configure their shared-memory attribute, build tensor
  maps' driver entry point and fill caches on their first launch;
* inputs live in static tensors that are overwritten in place before each replay; outputs are read from the tensors
  the capture produced;
* quantities that are passed to kernels BY VALUE are frozen at capture time (optimizer step counts for bias
  correction, learning rates, communication epochs), so optimizer steps and multi-GPU collectives stay outside the
  graph.  Forward and forward + backward passes of a single GPU are the intended use.

The reference has no counterpart (it launches every Triton kernel from Python).
"""
import torch

from ..tensor import Tensor


class CUDAGraph:
    """Thin handle: `capture_begin / capture_end / replay` like `torch.cuda.CUDAGraph`, usable with `graph(...)`."""

    def __init__(self):
        self._g = torch.cuda.CUDAGraph()

    def replay(self):
        self._g.replay()

    def reset(self):
        self._g.reset()


class graph:
    """Context manager: everything launched inside goes into `cuda_graph` instead of running."""

    def __init__(self, cuda_graph, pool=None, stream=None):
        self._ctx = torch.cuda.graph(cuda_graph._g, pool=pool, stream=stream)

    def __enter__(self):
        return self._ctx.__enter__()

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)


def _raw(x):
    return x._t if isinstance(x, Tensor) else x


class GraphedCallable:
    """`fn(*static_inputs)` captured once; calling the object copies new inputs into the static buffers, replays the
    graph and returns the static outputs (valid until the next call)."""

    def __init__(self, fn, sample_inputs, warmup=3):
        self.static_inputs = [Tensor._wrap(_raw(x).clone()) if isinstance(x, (Tensor, torch.Tensor)) else x
                              for x in sample_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = CUDAGraph()
        with graph(self.graph):
            self.static_outputs = fn(*self.static_inputs)

    def __call__(self, *inputs):
        for dst, src in zip(self.static_inputs, inputs):
            if isinstance(dst, Tensor):
                dst._t.copy_(_raw(src), non_blocking=True)
        self.graph.replay()
        return self.static_outputs


def make_graphed_callable(fn, sample_inputs, warmup=3):
    return GraphedCallable(fn, sample_inputs, warmup)

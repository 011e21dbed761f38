"""CUDA graphs for launch-bound loops: capture a fixed sequence of the framework's kernels once, replay it with one
launch.

The native kernels are launched on torch's current stream with plain runtime launches, and temporaries come from
torch's (or the native pool's) stream-ordered allocator, so a region that does no host read (`.item()`, `.numpy()`,
`check_status`) and changes no launch arguments between replays is capturable as is.  Rules of use:

* run the region eagerly a few times first (`warmup`): kernels configure their shared-memory attribute, build tensor
  maps' driver entry point and fill caches on their first launch;
* inputs live in static tensors that are overwritten in place before each replay; outputs are read from the tensors
  the capture produced;
* quantities that are passed to kernels BY VALUE are frozen at capture time (dropout seeds, communication epochs),
  so multi-GPU collectives and dropout stay outside a graph.  Adam/AdamW keep their step count, bias corrections and
  learning rate in a device vector once `make_capturable()` was called, which is what `GraphedTrainStep` does: a
  whole single-GPU training step (forward, backward, optimizer) replays as one launch.

The reference has no counterpart (it launches every Triton kernel from Python).
"""
import torch

from ..tensor import Tensor


class CUDAGraph:
    """Thin handle: `capture_begin / capture_end / replay` like `torch.cuda.CUDAGraph`, usable with `graph(...)`."""

    def __init__(self):
        self._g = torch.cuda.CUDAGraph()
        self._pool_capture = (0, 0)      # (device, id) of the native pool's private block list for this graph

    def replay(self):
        self._g.replay()

    def reset(self):
        self._g.reset()
        self._release_pool()

    def _release_pool(self):
        dev, cid = self._pool_capture
        if cid:
            from . import pool
            torch.cuda.synchronize(dev)
            pool.release_capture(dev, cid)
            self._pool_capture = (0, 0)

    def __del__(self):
        try:
            self._release_pool()
        except Exception:
            pass


class graph:
    """Context manager: everything launched inside goes into `cuda_graph` instead of running."""

    def __init__(self, cuda_graph, pool=None, stream=None):
        # "relaxed": pinned staging blocks for pointer tables may be allocated while capturing
        self._ctx = torch.cuda.graph(cuda_graph._g, pool=pool, stream=stream, capture_error_mode="relaxed")
        self._graph = cuda_graph

    def __enter__(self):
        from ..ops import native
        from . import pool as native_pool
        native.begin_capture_arena()          # pinned memory for pointer tables, reserved before the capture starts
        r = self._ctx.__enter__()
        # the native pool keeps what is allocated from here on out of eager code's reach for the graph's lifetime
        self._dev = torch.cuda.current_device()
        self._cid = native_pool.begin_capture(self._dev)
        return r

    def __exit__(self, *exc):
        from . import pool as native_pool
        if self._cid:
            native_pool.end_capture(self._dev)
            self._graph._pool_capture = (self._dev, self._cid)
        return self._ctx.__exit__(*exc)


def _raw(x):
    return x._t if isinstance(x, Tensor) else x


class GraphedCallable:
    """`fn(*static_inputs)` captured once; calling the object copies new inputs into the static buffers, replays the
    graph and returns the static outputs (valid until the next call)."""

    def __init__(self, fn, sample_inputs, warmup=3, warmup_inputs=None):
        self.static_inputs = [Tensor._wrap(_raw(x).clone()) if isinstance(x, (Tensor, torch.Tensor)) else x
                              for x in sample_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(warmup):
                if warmup_inputs is not None:        # eager calls on caller-supplied inputs (real batches)
                    self._load(warmup_inputs[i])
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = CUDAGraph()
        with graph(self.graph):
            self.static_outputs = fn(*self.static_inputs)

    def _load(self, inputs):
        for dst, src in zip(self.static_inputs, inputs):
            if isinstance(dst, Tensor):
                dst._t.copy_(_raw(src), non_blocking=True)

    def __call__(self, *inputs):
        self._load(inputs)
        self.graph.replay()
        return self.static_outputs


def make_graphed_callable(fn, sample_inputs, warmup=3):
    return GraphedCallable(fn, sample_inputs, warmup)


class GraphedTrainStep(GraphedCallable):
    """A whole training step as one CUDA graph.

    `step_fn(*inputs)` runs forward, backward and `optimizer.step()` (with `zero_grad`, and a `GradScaler` if one is
    used) and returns the loss.  The `warmup` eager calls are real training steps, on `warmup_inputs[i]` when that
    list of input tuples is given (real batches) and on `sample_inputs` otherwise; after them
    the step is captured once and every call replays it: inputs are copied into the static buffers, a changed
    `optimizer.lr` is written to the optimizer's device vector, and the returned loss is the static tensor the
    capture produced (valid until the next call).  Gradients stay readable in `p.grad` after a replay.
    Restrictions: fixed input shapes, no host reads inside `step_fn`, no dropout, one GPU.
    """

    def __init__(self, step_fn, optimizer, sample_inputs, warmup=3, warmup_inputs=None):
        if not hasattr(optimizer, "make_capturable"):
            raise TypeError("GraphedTrainStep needs an Adam / AdamW optimizer (device-resident step state)")
        optimizer.make_capturable()
        self.optimizer = optimizer
        from ..ops import native
        before = native.launch_count
        super().__init__(step_fn, sample_inputs, warmup, warmup_inputs)
        # kernels per replay = launches recorded while capturing (the last of warmup + 1 runs of step_fn)
        self.kernels_per_step = (native.launch_count - before) // (warmup + 1)
        optimizer.t -= 1          # the captured call counted a step that did not run

    def __call__(self, *inputs):
        self.optimizer._sync_lr()
        out = super().__call__(*inputs)
        self.optimizer.t += 1
        return out

"""Collective API. Parity: reference `genesis/distributed/nccl_backend.py:95-204` (signatures;
`async_op` accepted), with real all-gather / reduce-scatter instead of the reference's
broadcast loop and all-reduce-and-slice emulations.

CUDA float tensors with op SUM go to the peer-memory all-reduce kernel (in-kernel NVLink
loads/stores over the symmetric heap, no NCCL call) when `GENESIS_COMM` is `p2p` (default);
everything else, and `GENESIS_COMM=nccl`, uses the NCCL/gloo communicator.
"""
import os
from enum import Enum

import torch
import torch.distributed as tdist

from ..tensor import Tensor
from . import process_group as pg


class ReduceOp(Enum):
    SUM = "sum"
    PRODUCT = "product"
    MAX = "max"
    MIN = "min"
    BAND = "band"
    BOR = "bor"
    BXOR = "bxor"


_TORCH_OP = {ReduceOp.SUM: tdist.ReduceOp.SUM, ReduceOp.PRODUCT: tdist.ReduceOp.PRODUCT,
             ReduceOp.MAX: tdist.ReduceOp.MAX, ReduceOp.MIN: tdist.ReduceOp.MIN}


def _raw(t):
    return t._t if isinstance(t, Tensor) else t


def _op(op):
    if op not in _TORCH_OP:
        raise ValueError(f"Unsupported reduce op: {op}")
    return _TORCH_OP[op]


def comm_mode():
    return os.environ.get("GENESIS_COMM", "p2p").lower()


def _wrap_errors(fn, *a, **k):
    try:
        return fn(*a, **k)
    except RuntimeError as e:
        msg = str(e)
        low = msg.lower()
        if "timeout" in low or "timed out" in low:
            raise pg.CommTimeout(msg) from e
        raise


def all_reduce(tensor, op=ReduceOp.SUM, async_op=False):
    pg._check()
    if pg._world_size == 1:
        return None
    t = _raw(tensor)
    if t.is_cuda and op is ReduceOp.SUM and comm_mode() == "p2p" and t.dtype in (
            torch.float32, torch.bfloat16, torch.float16) and t.is_contiguous():
        from . import symm
        if symm.all_reduce_(t):
            return None
    _wrap_errors(tdist.all_reduce, t, op=_op(op))
    return None


def broadcast(tensor, src=0, async_op=False):
    pg._check()
    if pg._world_size == 1:
        return None
    t = _raw(tensor)
    if t.is_cuda and comm_mode() == "p2p":
        from . import symm
        if symm.broadcast_(t, src):
            return None
    _wrap_errors(tdist.broadcast, t, src=src)
    return None


def all_gather(tensor_list, tensor, async_op=False):
    """Fills `tensor_list[r]` with rank r's `tensor`."""
    pg._check()
    t = _raw(tensor)
    if pg._world_size == 1:
        _raw(tensor_list[0]).copy_(t)
        return None
    if t.is_cuda and comm_mode() == "p2p":
        from . import symm
        if symm.all_gather_([_raw(x) for x in tensor_list], t.contiguous()):
            return None
    _wrap_errors(tdist.all_gather, [_raw(x) for x in tensor_list], t.contiguous())
    return None


def reduce_scatter(output, input_list, op=ReduceOp.SUM, async_op=False):
    """output = reduce over ranks of input_list[my_rank]."""
    pg._check()
    out = _raw(output)
    if pg._world_size == 1:
        out.copy_(_raw(input_list[0]))
        return None
    ins = [_raw(x).contiguous() for x in input_list]
    if out.is_cuda and op is ReduceOp.SUM and comm_mode() == "p2p":
        from . import symm
        if symm.reduce_scatter_(out, ins):
            return None
    if pg._backend == "gloo":
        # gloo has no reduce_scatter: reduce the concatenation and keep our slice
        flat = torch.stack(ins)
        _wrap_errors(tdist.all_reduce, flat, op=_op(op))
        out.copy_(flat[pg._rank])
    else:
        _wrap_errors(tdist.reduce_scatter, out, ins, op=_op(op))
    return None


def all_to_all_single(output, input, output_split_sizes=None, input_split_sizes=None):
    pg._check()
    out, inp = _raw(output), _raw(input)
    if pg._world_size == 1:
        out.copy_(inp)
        return None
    if pg._backend == "gloo":
        W = pg._world_size
        ins = list(inp.split(input_split_sizes if input_split_sizes is not None else inp.shape[0] // W))
        outs = list(out.split(output_split_sizes if output_split_sizes is not None else out.shape[0] // W))
        reqs = []
        for r in range(W):
            if r == pg._rank:
                outs[r].copy_(ins[r])
            else:
                reqs.append(tdist.isend(ins[r].contiguous(), r))
                reqs.append(tdist.irecv(outs[r], r))
        for q in reqs:
            q.wait()
    else:
        if out.is_cuda and comm_mode() == "p2p" and inp.dim() >= 1:
            from . import symm
            W = pg._world_size
            ins = list(input_split_sizes) if input_split_sizes is not None else [inp.shape[0] // W] * W
            outs = list(output_split_sizes) if output_split_sizes is not None else [out.shape[0] // W] * W
            if symm.all_to_all_(out, inp.contiguous(), outs, ins):
                return None
        _wrap_errors(tdist.all_to_all_single, out, inp, output_split_sizes, input_split_sizes)
    return None


def barrier():
    pg._check()
    if pg._world_size == 1:
        return
    if comm_mode() == "p2p" and pg._backend == "nccl":
        from . import symm
        if symm.barrier_():
            return
    _wrap_errors(tdist.barrier)

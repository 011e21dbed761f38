"""Expert parallelism for `MoELayer`: experts are sharded over the ranks of a group and tokens
travel to their experts and back with two all-to-alls per layer and direction.

The reference has no expert parallelism at all (its MoE loops over every expert on one GPU,
`genesis/models/transformers/moe.py:317-361`).  Data flow of one layer on rank r:

    router -> sort (token, slot) pairs by global expert id  (= by destination rank)
           -> exchange per-expert counts                     (tiny all-to-all)
           -> dispatch rows to the owners of their experts   (all-to-all #1)
           -> regroup received rows expert-major, grouped SwiGLU GEMMs over local experts
           -> return rows to their source ranks               (all-to-all #2)
           -> weighted sum over the k slots of every token

Backward mirrors it through the same two all-to-alls in reverse.  Two transports implement
the row exchange: the communicator's `all_to_all_single` (NCCL / gloo; needs the split sizes
on the host), and on CUDA the peer-memory kernels of `csrc/moe_comm.cu`, which write rows
straight into the owner's receive buffer over NVLink from inside the dispatch kernel and need
no host synchronisation.  Expert parameters are marked `_no_ddp` so `DistributedDataParallel`
does not all-reduce them; it scales their gradients by 1/world instead (every rank's loss is a
local mean and the experts see tokens of all ranks).
"""
import torch

from ..distributed import process_group as pg
from ..distributed import collectives as C
from ..function import Function, AMPPolicy
from ..ops import dispatch as K
from ..tensor import Tensor


class EPGroup:
    """The expert-parallel group: all ranks of the process group."""

    def __init__(self):
        self.size = pg.get_world_size() if pg.is_initialized() else 1
        self.rank = pg.get_rank() if pg.is_initialized() else 0


class AllToAllRows(Function):
    """Rows of `x` split by `send_splits` go to the ranks; `recv_splits` rows come back."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, send_splits, recv_splits):
        ctx.splits = (send_splits, recv_splits)
        out = torch.empty(sum(recv_splits), x.shape[1], dtype=x.dtype, device=x.device)
        C.all_to_all_single(out, x.contiguous(), recv_splits, send_splits)
        return out

    @staticmethod
    def backward(ctx, g):
        send_splits, recv_splits = ctx.splits
        out = torch.empty(sum(send_splits), g.shape[1], dtype=g.dtype, device=g.device)
        C.all_to_all_single(out, g.contiguous(), send_splits, recv_splits)
        return out


class PermuteRows(Function):
    """out[i] = x[src[i]] for a permutation `src`."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, src):
        ctx.save_for_backward(src)
        return K.gather_rows(x, src)

    @staticmethod
    def backward(ctx, g):
        (src,) = ctx.saved_tensors
        out = torch.empty_like(g)
        out[src] = g
        return out


def mark_expert_parameters(model):
    """Flag expert-sharded parameters so DDP leaves them out of its buckets."""
    from ..models.transformers.moe import GroupedExperts
    n = 0
    for m in model.modules():
        if isinstance(m, GroupedExperts) and m.total_experts != m.num_experts:
            for p in (m.w_gate, m.w_up, m.w_down):
                p._no_ddp = True
                n += 1
    return n


def expert_parallel_forward(layer, x, idx, w):
    """x Tensor [T, H]; idx raw int tensor [T, k] (global expert ids); w Tensor [T, k]."""
    from ..models.transformers.moe import DispatchFunction, CombineFunction
    ep = layer.ep
    W, E = ep.size, layer.num_experts
    El = E // W
    T, k = idx.shape
    dev = idx.device
    token_of, pos, offsets = K.moe_sort_unpadded(idx, E)          # sorted by global expert id = by destination rank
    xs = DispatchFunction.apply(x, Tensor._wrap(token_of))

    send_counts = (offsets[1:] - offsets[:-1]).to(torch.int64)             # [E] rows per global expert
    recv_counts = torch.empty(W * El, dtype=torch.int64, device=dev)       # [W, El] rows from rank r for local e
    C.all_to_all_single(recv_counts, send_counts)
    send_splits = send_counts.reshape(W, El).sum(1).tolist()
    rc = recv_counts.reshape(W, El)
    recv_splits = rc.sum(1).tolist()

    xr = AllToAllRows.apply(xs, send_splits, recv_splits)                 # rank-major, expert-minor
    # regroup expert-major: row order key = (local expert, source rank)
    R = int(sum(recv_splits))
    seg_expert = torch.arange(El, device=dev).repeat(W)                    # expert id of each (r, e) segment
    row_expert = torch.repeat_interleave(seg_expert, rc.reshape(-1), output_size=R)
    order = torch.sort(row_expert, stable=True)[1]
    local_offsets = torch.zeros(El + 1, dtype=torch.int64, device=dev)
    local_offsets[1:] = torch.cumsum(rc.sum(0), 0)
    xe = PermuteRows.apply(xr, Tensor._wrap(order))
    ye = layer.experts(xe, local_offsets)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(R, device=dev, dtype=order.dtype)
    yr = PermuteRows.apply(ye, Tensor._wrap(inv))                          # back to rank-major order
    ys = AllToAllRows.apply(yr, recv_splits, send_splits)                 # back on the source rank, sorted order
    return CombineFunction.apply(ys, w, Tensor._wrap(pos))

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
on the host), and on CUDA (`GENESIS_COMM=p2p`, the default) the peer-memory kernels of
`csrc/moe_comm.cu`: the owner of an expert pulls the rows it needs straight out of the source
ranks' activation buffers over NVLink, and the source rank pulls the expert outputs back while it
forms the weighted sum, with no host synchronisation anywhere in the layer.  Expert parameters are marked `_no_ddp` so `DistributedDataParallel`
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
            for p in (m.w_gate_up, m.w_down):
                p._no_ddp = True
                n += 1
    return n


# ---------------------------------------------------------------------------------------------
# peer-memory transport
# ---------------------------------------------------------------------------------------------
class _Workspace:
    """Symmetric buffers of the pull kernels, allocated collectively on first use and regrown (on every rank at
    once: shapes are the same everywhere) when a larger layer shows up."""

    def __init__(self):
        self.key = None

    def ensure(self, T, k, H, cap, dtype):
        from ..distributed import symm
        es = torch.empty(0, dtype=dtype).element_size()
        key = (T, k, H, cap, es)
        if self.key is not None and all(a <= b for a, b in zip(key, self.key)):
            return
        self.key = key
        self.x = symm.alloc(T * H * es)          # forward: token rows
        self.g = symm.alloc(T * H * es)          # backward: gradient of the layer output
        self.tok = symm.alloc(T * k * 4)
        self.ws = symm.alloc(T * k * 4)
        self.y = symm.alloc(cap * H * es)        # forward: expert outputs in the owner's layout
        self.dx = symm.alloc(cap * H * es)       # backward: gradient of the received rows
        self.dwr = symm.alloc(cap * 4)


_ws = _Workspace()
_CTAS = 128             # CTAs of the pull kernels (the same on every rank: each CTA has its own flag channel)


def _stage_rows(rows, buf, sh, H):
    """Copies the rows of the receive layout that exist into a symmetric buffer (count read on the device)."""
    from ..ops import native as N
    N._chk(N.lib().gb_ep_stage_rows(rows.data_ptr(), buf.local_ptr, sh["local_offsets"][sh["El"]:].data_ptr(),
                                    H * rows.element_size(), sh["cap"], N._st()), "ep_stage_rows")

p2p_layers_run = 0      # forward passes that took the peer-memory transport (tests assert on it)

# Optional device timing of the pull kernels (CUDA events around every dispatch / combine launch, forward and
# backward): `profile_comm(True)` switches it on, `comm_profile()` reads it back.
_prof = {"on": False, "events": []}


def profile_comm(on=True):
    _prof["on"] = bool(on)
    _prof["events"] = []


class _Timed:
    def __init__(self, kind, nbytes):
        self.kind, self.nbytes = kind, nbytes

    def __enter__(self):
        if _prof["on"]:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e1 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if _prof["on"]:
            self.e1.record()
            _prof["events"].append((self.kind, self.nbytes, self.e0, self.e1))
        return False


def comm_profile(link_gbs=900.0):
    """Per-call device time of the dispatch / combine pull kernels since `profile_comm(True)`, the bytes each call
    moves over NVLink into this rank ((W - 1) / W of the rows for a balanced router) and the fraction of the link
    bound (bytes / `link_gbs`) that time represents.  Synchronises."""
    if not _prof["events"]:
        return None
    torch.cuda.synchronize()
    out = {}
    for kind in ("dispatch", "combine"):
        ev = [(b, e0.elapsed_time(e1)) for k, b, e0, e1 in _prof["events"] if k == kind]
        if not ev:
            continue
        ms = sorted(t for _, t in ev)[len(ev) // 2]
        nb = ev[0][0]
        bound_ms = nb / (link_gbs * 1e9) * 1e3
        out[kind] = {"calls": len(ev), "ms_per_call_median": ms, "nvlink_bytes_per_call": nb,
                     "bound_ms_at_%d_gbs" % int(link_gbs): bound_ms, "fraction_of_bound": bound_ms / ms if ms else None}
    return out


def _p2p_usable(x):
    from ..distributed import symm
    return x.is_cuda and C.comm_mode() == "p2p" and symm.available() and x.dtype in (
        torch.bfloat16, torch.float16, torch.float32)


class EPDispatchPull(Function):
    """xe[row] = x_p[token] for every (token, slot) pair routed to a local expert, pulled over peer memory into the
    padded expert-major layout.  `w` rides along so that its gradient, which the owners of the experts compute,
    can be returned here."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, x, w, idx, shared):
        from ..distributed import symm
        from ..ops import native as N
        from ..ops import grouped
        st = symm.state()
        W, E, El = shared["W"], shared["E"], shared["El"]
        T, k = idx.shape
        H = x.shape[1]
        dev = x.device
        cap = shared["cap"]
        _ws.ensure(T, k, H, cap, x.dtype)
        token_of, pos, offsets = K.moe_sort_unpadded(idx, E)      # int32: sorted by global expert = by owner
        token_of = token_of.to(torch.int32)
        pos = pos.to(torch.int32).contiguous()
        offsets = offsets.to(torch.int32).contiguous()
        _ws.x.view(x.dtype, 0, T * H).copy_(x.reshape(-1))
        _ws.tok.view(torch.int32, 0, T * k).copy_(token_of.reshape(-1))
        all_off = [torch.empty(E + 1, dtype=torch.int32, device=dev) for _ in range(W)]
        if not symm.all_gather_(all_off, offsets):
            raise RuntimeError("peer-memory all-gather unavailable")
        all_off = torch.stack(all_off).contiguous()
        local_offsets = torch.empty(El + 1, dtype=torch.int32, device=dev)
        seg_start = torch.empty(El * W, dtype=torch.int32, device=dev)
        seg_src = torch.empty(El * W, dtype=torch.int32, device=dev)
        dest_base = torch.empty(E, dtype=torch.int32, device=dev)
        info = torch.zeros(2, dtype=torch.int32, device=dev)
        L = N.lib()
        N._chk(L.gb_ep_layout(all_off.data_ptr(), st.rank, W, E, grouped.ALIGN, cap, local_offsets.data_ptr(),
                              seg_start.data_ptr(), seg_src.data_ptr(), dest_base.data_ptr(), info.data_ptr(),
                              st.status.data_ptr(), N._st()), "ep_layout")
        xe = torch.empty(cap, H, dtype=x.dtype, device=dev)     # rows past the layout's end stay unwritten
        remote = T * k * H * x.element_size() * (W - 1) // W       # bytes a balanced router sends over NVLink
        sh_timer = _Timed("dispatch", remote)
        sh_timer.__enter__()
        N._chk(L.gb_ep_dispatch_pull(_ws.x.ptr_table, _ws.tok.ptr_table, None, st.flags.ptr_table, all_off.data_ptr(),
                                     local_offsets.data_ptr(), seg_start.data_ptr(), seg_src.data_ptr(), xe.data_ptr(),
                                     None, None, H, st.rank, W, E, cap, 0, symm.next_epoch(), N._DT[x.dtype], _CTAS,
                                     N._comm_budget(), st.status.data_ptr(), N._st()), "ep_dispatch_pull")
        sh_timer.__exit__()
        shared.update(token_of=token_of, pos=pos, offsets=offsets, all_off=all_off, local_offsets=local_offsets,
                      seg_start=seg_start, seg_src=seg_src, dest_base=dest_base, T=T, k=k, H=H)
        ctx.shared = shared
        ctx.w_dtype = w.dtype
        return xe

    @staticmethod
    def backward(ctx, g):
        from ..distributed import symm
        from ..ops import native as N
        sh = ctx.shared
        st = symm.state()
        T, k, H, cap = sh["T"], sh["k"], sh["H"], sh["cap"]
        g = g if g.is_contiguous() else g.contiguous()
        _stage_rows(g, _ws.dx, sh, H)
        _ws.dwr.view(torch.float32, 0, cap).copy_(sh["dwr"])
        dx = torch.empty(T, H, dtype=g.dtype, device=g.device)
        dw = torch.empty(T, k, dtype=torch.float32, device=g.device)
        tm = _Timed("combine", T * k * H * g.element_size() * (sh["W"] - 1) // sh["W"])
        tm.__enter__()
        N._chk(N.lib().gb_ep_combine_pull(_ws.dx.ptr_table, _ws.dwr.ptr_table, st.flags.ptr_table,
                                          sh["idx"].data_ptr(), sh["pos"].data_ptr(), None, sh["offsets"].data_ptr(),
                                          sh["dest_base"].data_ptr(), dx.data_ptr(), dw.data_ptr(), T, k, H, st.rank,
                                          sh["W"], sh["E"], cap, 1, symm.next_epoch(), N._DT[g.dtype], _CTAS,
                                          N._comm_budget(), st.status.data_ptr(), N._st()), "ep_combine_pull(bwd)")
        tm.__exit__()
        return dx, dw.to(ctx.w_dtype)


class EPCombinePull(Function):
    """out[t] = sum_j w[t, j] * ye_owner[row(t, j)], pulled from the owners' output buffers."""
    raw = True
    amp_policy = AMPPolicy.PRESERVE

    @staticmethod
    def forward(ctx, ye, w, shared):
        from ..distributed import symm
        from ..ops import native as N
        sh = shared
        st = symm.state()
        T, k, H, cap = sh["T"], sh["k"], sh["H"], sh["cap"]
        ye = ye if ye.is_contiguous() else ye.contiguous()
        _stage_rows(ye, _ws.y, sh, H)
        wf = w.to(torch.float32).contiguous()
        out = torch.empty(T, H, dtype=ye.dtype, device=ye.device)
        W = sh["W"]
        tm = _Timed("combine", T * k * H * ye.element_size() * (W - 1) // W)
        tm.__enter__()
        N._chk(N.lib().gb_ep_combine_pull(_ws.y.ptr_table, None, st.flags.ptr_table, sh["idx"].data_ptr(),
                                          sh["pos"].data_ptr(), wf.data_ptr(), sh["offsets"].data_ptr(),
                                          sh["dest_base"].data_ptr(), out.data_ptr(), None, T, k, H, st.rank, sh["W"],
                                          sh["E"], cap, 0, symm.next_epoch(), N._DT[ye.dtype], _CTAS, N._comm_budget(),
                                          st.status.data_ptr(), N._st()), "ep_combine_pull")
        tm.__exit__()
        ctx.shared = sh
        ctx.save_for_backward(ye, wf)
        return out

    @staticmethod
    def backward(ctx, g):
        from ..distributed import symm
        from ..ops import native as N
        sh = ctx.shared
        ye, wf = ctx.saved_tensors
        st = symm.state()
        T, k, H, cap = sh["T"], sh["k"], sh["H"], sh["cap"]
        g = g if g.dtype == ye.dtype else K.to_dtype(g, ye.dtype)
        _ws.g.view(g.dtype, 0, T * H).copy_(g.reshape(-1))
        _ws.tok.view(torch.int32, 0, T * k).copy_(sh["token_of"].reshape(-1))
        # routing weight of every pair, in sorted-pair order
        ws_sorted = _ws.ws.view(torch.float32, 0, T * k)
        ws_sorted[sh["pos"].reshape(-1).long()] = wf.reshape(-1)
        dye = torch.empty(cap, H, dtype=ye.dtype, device=ye.device)
        dwr = torch.zeros(cap, dtype=torch.float32, device=ye.device)
        tm = _Timed("dispatch", T * k * H * ye.element_size() * (sh["W"] - 1) // sh["W"])
        tm.__enter__()
        N._chk(N.lib().gb_ep_dispatch_pull(_ws.g.ptr_table, _ws.tok.ptr_table, _ws.ws.ptr_table, st.flags.ptr_table,
                                           sh["all_off"].data_ptr(), sh["local_offsets"].data_ptr(),
                                           sh["seg_start"].data_ptr(), sh["seg_src"].data_ptr(), dye.data_ptr(),
                                           ye.data_ptr(), dwr.data_ptr(), H, st.rank, sh["W"], sh["E"], cap, 1,
                                           symm.next_epoch(), N._DT[ye.dtype], _CTAS, N._comm_budget(),
                                           st.status.data_ptr(), N._st()), "ep_dispatch_pull(bwd)")
        tm.__exit__()
        sh["dwr"] = dwr
        return dye, None


def _expert_parallel_forward_p2p(layer, x, idx, w):
    import os
    from ..ops import grouped
    global p2p_layers_run
    p2p_layers_run += 1
    ep = layer.ep
    W, E = ep.size, layer.num_experts
    El = E // W
    T, k = idx.shape
    # receive buffers are sized for `factor` times the balanced share; a freshly initialised router is skewed (2.1x
    # was seen on 8 ranks), and rows beyond the buffer raise an error instead of being dropped
    factor = float(os.environ.get("GENESIS_EP_CAPACITY", min(W, 4.0 if W > 2 else 2.0)))
    cap = (int(factor * T * k) + grouped.ALIGN - 1) // grouped.ALIGN * grouped.ALIGN + El * grouped.ALIGN
    shared = {"W": W, "E": E, "El": El, "cap": cap, "idx": idx.to(torch.int32).contiguous()}
    xe = EPDispatchPull.apply(x, w, shared["idx"], shared)
    ye = layer.experts(xe, shared["local_offsets"])
    return EPCombinePull.apply(ye, w.detach(), shared)


def expert_parallel_forward(layer, x, idx, w):
    """x Tensor [T, H]; idx raw int tensor [T, k] (global expert ids); w Tensor [T, k]."""
    from ..models.transformers.moe import DispatchFunction, CombineFunction
    if _p2p_usable(x._t):
        return _expert_parallel_forward_p2p(layer, x, idx, w)
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

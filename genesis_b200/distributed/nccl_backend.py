"""`genesis.distributed.nccl_backend.NCCLBackend` of the reference: an object with `init_process_group / destroy /
barrier / all_reduce / all_gather / broadcast / reduce_scatter`.  The reference binds libnccl through ctypes and
exchanges the unique id over its own TCP server; here NCCL is reached through `torch.distributed` (the baseline
transport of this framework, `GENESIS_COMM=nccl`), and the object delegates to the package-level API, so that the
peer-memory kernels serve it too when they are the selected transport."""
from . import collectives as _C
from . import process_group as _pg
from .collectives import ReduceOp


class NCCLBackend:
    def __init__(self):
        self.initialized = False
        self.rank = 0
        self.world_size = 1

    def init_process_group(self, init_method, world_size, rank):
        _pg.init_process_group("nccl", init_method=init_method, world_size=world_size, rank=rank)
        self.initialized = True
        self.rank, self.world_size = _pg.get_rank(), _pg.get_world_size()

    def destroy(self):
        if self.initialized:
            _pg.destroy_process_group()
            self.initialized = False

    def barrier(self):
        return _C.barrier()

    def all_reduce(self, tensor, op=ReduceOp.SUM, async_op=False):
        return _C.all_reduce(tensor, op, async_op)

    def all_gather(self, tensor_list, tensor, async_op=False):
        return _C.all_gather(tensor_list, tensor, async_op)

    def broadcast(self, tensor, src, async_op=False):
        return _C.broadcast(tensor, src, async_op)

    def reduce_scatter(self, output, input_list, op=ReduceOp.SUM, async_op=False):
        return _C.reduce_scatter(output, input_list, op, async_op)

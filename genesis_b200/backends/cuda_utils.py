"""`genesis.backends.cuda_utils` of the reference: storage constructors."""
from .cuda import empty, ones, zeros  # noqa: F401


def set_cuda_storage_factory(factory):
    """Accepted for API parity: storages of this framework are always `CUDAStorage` over pool-allocated tensors."""
    return None

"""`import genesis` (the alias package) and the reference's top-level import surface
(`genesis/__init__.py:9-72`: `from .backends import *`, `from .functional import *`)."""
import numpy as np
import torch


def test_alias_is_the_same_module_tree():
    import genesis
    import genesis_b200
    assert genesis is genesis_b200
    import genesis.nn.functional as F
    import genesis_b200.nn.functional as F2
    assert F is F2
    from genesis.models.transformers.moe import MoELayer
    from genesis_b200.models.transformers.moe import MoELayer as M2
    assert MoELayer is M2
    from genesis.backends import Storage, CPUStorage, CUDAStorage      # noqa: F401
    from genesis.nn.triton_ops import fused_rmsnorm, safe_softmax      # noqa: F401
    from genesis.nn.attention import FusedAttention, fused_attention    # noqa: F401
    from genesis.nn.layer_norm import fused_layer_norm                  # noqa: F401


def test_star_exported_functional_names():
    import genesis
    names = """cross_entropy sparse_cross_entropy dropout gelu silu scaled_dot_product_attention view expand flatten
        contiguous broadcast_to clip t floordiv multiply divide negate summation sum_to_shape getitem setitem
        add_scalar sub_scalar mul_scalar divide_scalar pow_scalar add_inplace sub_inplace mul_inplace truediv
        EWiseAdd EWiseSub EWiseMul EWiseDiv AddScalar SubScalar MulScalar DivScalar PowScalar Negate Sin Cos Log Exp
        Sqrt Abs Clamp Where Permute Transpose Reshape Expand View Flatten BroadcastTo Summation Mean Matmul ReLU
        LogSumExp Max Min Stack Cat Squeeze Unsqueeze Split Sigmoid Tanh Maximum Gather Scatter SetItem
        GetItemView GetItemGather TopKFunction ScatterAddFunction RepeatInterleaveFunction FusedAttention
        FusedLayerNormFunction fused_layer_norm fused_attention safe_softmax CastFP32 cast_fp32 Equal Argmax Argmin
        Norm Contiguous Storage CPUStorage CUDAStorage triu tril argsort sort bincount nonzero allclose eq ne gt ge
        lt le isinf isnan isfinite""".split()
    missing = [n for n in names if not hasattr(genesis, n)]
    assert not missing, missing
    x = genesis.tensor(np.arange(6, dtype=np.float32).reshape(2, 3), requires_grad=True)
    y = genesis.summation(genesis.multiply(genesis.view(x, (3, 2)), 2.0))
    y.backward()
    np.testing.assert_allclose(x.grad.numpy(), 2.0)
    assert genesis.cross_entropy(x, genesis.tensor([0, 2], dtype=genesis.int64)).shape == ()
    assert genesis.EWiseAdd.apply(x, x).shape == (2, 3)


def test_all_any_allclose_return_tensors():
    import genesis
    x = genesis.tensor([1.0, 2.0, 0.0])
    assert not x.all().item() and x.any().item() and bool(x.any())
    m = genesis.tensor([[1.0, 0.0], [1.0, 1.0]])
    assert m.all(dim=1).numpy().tolist() == [False, True]
    assert m.any(dim=0, keepdim=True).shape == (1, 2)
    assert genesis.allclose(x, x).item() is True
    v, i = genesis.topk(genesis.tensor([3.0, 1.0]), k=5, dim=0)
    assert v.shape == (2,)


def test_storage_classes():
    import genesis
    from genesis.backends import CPUStorage
    from genesis.storage import Storage
    s = Storage.allocate((2, 3), genesis.float32)
    assert s.numel == 6 and s.shape == (2, 3) and s.dtype == "float32" and s.element_size() == 4
    m = Storage.make_storage(np.arange(4, dtype=np.float32))
    assert m.to_numpy().tolist() == [0, 1, 2, 3] and m[1] == 1.0
    c = CPUStorage(np.ones((2, 2), np.float32))
    assert isinstance(c, torch.Tensor) and c.clone().to_numpy().sum() == 4 and c.fill(3).to_numpy()[0, 0] == 3
    h = m.to_dtype("float16")
    assert h.dtype == "float16"


def test_reference_module_paths_and_small_interfaces():
    """Same-path modules of the reference that user code may import, and the small interfaces behind them."""
    import importlib
    import numpy as np
    for path in ("genesis.optim.adamw", "genesis.distributed.comm", "genesis.distributed.parallel",
                 "genesis.distributed.nccl_backend", "genesis.amp.amp_cache", "genesis.ops.dispatcher",
                 "genesis.backends.base", "genesis.backends.cpu", "genesis.backends.cuda_error",
                 "genesis.nn.triton_ops.rmsnorm", "genesis.nn.triton_ops.softmax", "genesis.nn.triton_ops.grad_check",
                 "genesis.nn.triton_ops.dropout", "genesis.nn.triton_ops.gelu", "genesis.nn.triton_ops.silu",
                 "genesis.nn.triton_ops.layer_norm"):
        importlib.import_module(path)
    import genesis
    from genesis.optim.adamw import AdamW
    from genesis.distributed.parallel import DistributedDataParallel
    from genesis.distributed.nccl_backend import NCCLBackend
    assert AdamW is genesis.optim.AdamW and DistributedDataParallel is genesis.nn.parallel.DistributedDataParallel
    assert not NCCLBackend().initialized
    from genesis.ops.dispatcher import OperationDispatcher, register_cpu

    @register_cpu("twice")
    def twice(x, bonus=0):
        return x * 2 + bonus
    t = genesis.tensor(np.ones(3, np.float32))
    assert OperationDispatcher.has_implementation("twice", "cpu") and not OperationDispatcher.has_implementation("twice", "cuda")
    assert np.allclose(OperationDispatcher.dispatch("twice", t, bonus=1).numpy(), 3.0)
    assert isinstance(OperationDispatcher.dispatch_tuple("twice", t), tuple)
    try:
        OperationDispatcher.dispatch("nothing", t)
        raise AssertionError("expected NotImplementedError")
    except NotImplementedError:
        pass
    from genesis.amp.amp_cache import get_amp_cache
    cache = get_amp_cache()
    cache.clear()
    cache.reset_stats()
    p = genesis.tensor(np.ones((2, 2), np.float32), requires_grad=True)
    a = cache.cached_cast(p, genesis.bfloat16)
    b = cache.cached_cast(p, genesis.bfloat16)
    assert a is b and a.dtype == genesis.bfloat16 and cache.get_stats()["hits"] == 1 and cache.get_stats()["misses"] == 1
    cache.clear()
    from genesis.backends.cuda_error import check_cuda_error
    assert check_cuda_error((0, 5)) == 5 and check_cuda_error(0) is None
    try:
        check_cuda_error((2,))
        raise AssertionError("expected RuntimeError")
    except RuntimeError:
        pass
    from genesis.nn.triton_ops.grad_check import check_finite_kernel
    import torch
    flag = torch.zeros(1)
    check_finite_kernel([genesis.tensor(np.array([1.0, np.inf], np.float32))], flag)
    assert float(flag) == 1.0

"""`genesis.ops.dispatcher` of the reference: a registry of per-device implementations.  The built-in operators of this
framework do not go through a registry (one function per op in `ops/dispatch.py`: CUDA -> native kernels, CPU -> torch);
this module keeps the reference's interface for user code that registers and dispatches its OWN operators by name."""
from typing import Any, Callable

_registry = {}


def _device_type(x):
    t = getattr(x, "_t", x)
    dev = getattr(t, "device", None)
    kind = getattr(dev, "type", None) or str(dev or "cpu")
    return "cuda" if "cuda" in str(kind) else "cpu"


class OperationDispatcher:
    @classmethod
    def register(cls, op_name: str, device_type, impl_func: Callable):
        _registry.setdefault(op_name, {})[_norm(device_type)] = impl_func

    @classmethod
    def has_implementation(cls, op_name: str, device_type) -> bool:
        return _norm(device_type) in _registry.get(op_name, {})

    @classmethod
    def _impl(cls, op_name, device_type):
        impls = _registry.get(op_name)
        if not impls:
            raise NotImplementedError(f"Operation '{op_name}' not registered")
        if device_type not in impls:
            raise NotImplementedError(f"Operation '{op_name}' not implemented for device {device_type}")
        return impls[device_type]

    @classmethod
    def dispatch(cls, op_name: str, *tensors, **kwargs) -> Any:
        if not tensors:
            raise ValueError(f"Operation '{op_name}' requires at least one tensor argument")
        return cls._impl(op_name, _device_type(tensors[0]))(*tensors, **kwargs)

    @classmethod
    def dispatch_inplace(cls, op_name: str, target_tensor, *args, **kwargs):
        cls._impl(op_name, _device_type(target_tensor))(target_tensor, *args, **kwargs)
        return target_tensor

    @classmethod
    def dispatch_tuple(cls, op_name: str, *tensors, **kwargs):
        out = cls.dispatch(op_name, *tensors, **kwargs)
        return out if isinstance(out, tuple) else (out,)

    @classmethod
    def dispatch_creation(cls, op_name: str, device, *args, **kwargs):
        return cls._impl(op_name, _norm(device))(*args, **kwargs)


def _norm(device_type):
    s = str(getattr(device_type, "name", None) or getattr(device_type, "type", None) or device_type).lower()
    return "cuda" if "cuda" in s else "cpu"


def register_cpu(op_name: str):
    def decorator(func: Callable):
        OperationDispatcher.register(op_name, "cpu", func)
        return func
    return decorator


def register_cuda(op_name: str):
    def decorator(func: Callable):
        OperationDispatcher.register(op_name, "cuda", func)
        return func
    return decorator

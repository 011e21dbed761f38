"""Checkpoint I/O. Parity: reference `genesis/serialization.py:6-73`.

The stream is a dill/pickle stream (protocol 4) in which every tensor is rebuilt by
`_rebuild_tensor(numpy_array, dtype_name, requires_grad)`.  Files written by the
reference name that hook `genesis.tensor._rebuild_tensor`; the loader maps the
`genesis.*` module paths onto this package, and `save(..., compat=True)` writes that
name, so checkpoints travel in both directions.  Unlike the reference
(`serialization.py:24-25`) `save` leaves the caller's dict intact, and the write is
atomic: temp file, fsync, `os.replace`; an existing file is kept as
`<path>.genesis.bak` until the new one is in place.
"""
import io
import os
import shutil
import sys
import types

import dill

from .tensor import Tensor as _Tensor, _rebuild_tensor as _rebuild


class _Unpickler(dill.Unpickler):
    def find_class(self, module, name):
        if module == "genesis" or module.startswith("genesis."):
            mapped = "genesis_b200" + module[len("genesis"):]
            try:
                return super().find_class(mapped, name)
            except (ImportError, AttributeError, ModuleNotFoundError):
                pass
        return super().find_class(module, name)


def _compat_dumps(obj):
    """Pickle with tensors referring to the global `genesis.tensor._rebuild_tensor`."""
    saved = {}
    mod = sys.modules.get("genesis.tensor")
    if mod is not None and getattr(getattr(mod, "_rebuild_tensor", None), "__module__", None) == "genesis.tensor":
        hook = mod._rebuild_tensor                  # the reference itself is loaded: its own hook
    else:
        # no `genesis` package, or the alias of this framework (whose hook pickles under this package's name):
        # stand-in modules for the duration of the dump, the previous entries put back afterwards
        src = _rebuild
        hook = types.FunctionType(src.__code__, src.__globals__, "_rebuild_tensor")
        hook.__module__ = "genesis.tensor"
        hook.__qualname__ = "_rebuild_tensor"
        pkg = types.ModuleType("genesis")
        pkg.__path__ = []
        sub = types.ModuleType("genesis.tensor")
        sub._rebuild_tensor = hook
        pkg.tensor = sub
        for k in ("genesis", "genesis.tensor"):
            saved[k] = sys.modules.get(k)
        sys.modules["genesis"], sys.modules["genesis.tensor"] = pkg, sub

    class CompatPickler(dill.Pickler):
        def reducer_override(self, o):
            if isinstance(o, _Tensor):
                return (hook, o.__reduce__()[1])
            return NotImplemented

    try:
        buf = io.BytesIO()
        CompatPickler(buf, protocol=4).dump(obj)
        return buf.getvalue()
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def save(state_dict, file_path, compat=False):
    """Write `state_dict` to `file_path` atomically.

    `compat=True` names the tensor hook as the reference does, so the reference's
    `genesis.load` can read the file.
    """
    file_path = os.fspath(file_path)
    backup = file_path + ".genesis.bak"
    had_old = os.path.exists(file_path)
    if had_old:
        shutil.copyfile(file_path, backup)
    tmp = file_path + ".tmp"
    try:
        data = _compat_dumps(state_dict) if compat else dill.dumps(state_dict, protocol=4)
        with open(tmp, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, file_path)
    except BaseException:
        if os.path.exists(tmp):
            os.remove(tmp)
        if had_old and os.path.exists(backup):
            shutil.copyfile(backup, file_path)
        raise
    finally:
        if os.path.exists(backup):
            os.remove(backup)


def load(file_path):
    with open(os.fspath(file_path), "rb") as f:
        return _Unpickler(f).load()


def save_checkpoint(model_state_dict, optimizer_state_dict, file_path, **extra):
    ckpt = {"model_state_dict": model_state_dict, "optimizer_state_dict": optimizer_state_dict}
    ckpt.update(extra)
    save(ckpt, file_path)


def load_checkpoint(file_path):
    ckpt = load(file_path)
    return ckpt["model_state_dict"], ckpt["optimizer_state_dict"]

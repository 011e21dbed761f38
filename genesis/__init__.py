"""`import genesis` for code written against phonism/genesis: the module object IS `genesis_b200`.

Every `genesis.x.y` import resolves to the already-loaded `genesis_b200.x.y` module (one copy of each
module, two names), so `import genesis.nn.functional as F`, `from genesis.backends import CUDAStorage`
or `from genesis.models.transformers.moe import MoELayer` work unchanged.
Import surface parity: reference `genesis/__init__.py:9-72`.
"""
import importlib
import importlib.abc
import importlib.util
import sys

import genesis_b200 as _impl

_SRC, _DST = "genesis_b200", __name__


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target):
        self._target = target

    def create_module(self, spec):
        return importlib.import_module(self._target)

    def exec_module(self, module):          # already executed under its real name
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    """Maps `genesis.<rest>` to `genesis_b200.<rest>`."""

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_DST + "."):
            return None
        real = _SRC + fullname[len(_DST):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError, AttributeError):
            return None
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real))


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
for _name, _mod in list(sys.modules.items()):
    if _name == _SRC or _name.startswith(_SRC + "."):
        sys.modules[_DST + _name[len(_SRC):]] = _mod
sys.modules[_DST] = _impl

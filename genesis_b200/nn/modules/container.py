"""`Sequential` and `ModuleList`. Parity: reference `genesis/nn/modules/container.py:8-89`."""
from .module import Module, ModuleContainer


class Sequential(ModuleContainer):
    """Children are keyed `0.`, `1.`, ... in the state dict."""

    def __init__(self, *modules):
        super().__init__()
        if len(modules) == 1 and isinstance(modules[0], (list, tuple)):
            modules = tuple(modules[0])
        self._modules_list = list(modules)

    def forward(self, x):
        for m in self._modules_list:
            x = m(x)
        return x

    def __getitem__(self, i):
        if isinstance(i, slice):
            return Sequential(*self._modules_list[i])
        return self._modules_list[i]

    def __len__(self):
        return len(self._modules_list)

    def __iter__(self):
        return iter(self._modules_list)

    def append(self, m):
        self._modules_list.append(m)
        return self


class ModuleList(ModuleContainer):
    """A list of modules; an attribute `layers = ModuleList(...)` yields keys `layers.0.…`."""

    def __init__(self, modules=None):
        super().__init__()
        self._modules_list = list(modules) if modules is not None else []

    def append(self, m):
        self._modules_list.append(m)
        return self

    def extend(self, ms):
        self._modules_list.extend(ms)
        return self

    def insert(self, i, m):
        self._modules_list.insert(i, m)

    def __getitem__(self, i):
        if isinstance(i, slice):
            return ModuleList(self._modules_list[i])
        return self._modules_list[i]

    def __setitem__(self, i, m):
        self._modules_list[i] = m

    def __len__(self):
        return len(self._modules_list)

    def __iter__(self):
        return iter(self._modules_list)

    def forward(self, *a, **k):
        raise NotImplementedError("ModuleList is not callable")


class ModuleDict(ModuleContainer):
    _list_attr = "_modules_dict"

    def __init__(self, modules=None):
        super().__init__()
        self._modules_dict = dict(modules) if modules is not None else {}

    def __getitem__(self, k):
        return self._modules_dict[k]

    def __setitem__(self, k, m):
        self._modules_dict[k] = m

    def __contains__(self, k):
        return k in self._modules_dict

    def __len__(self):
        return len(self._modules_dict)

    def __iter__(self):
        return iter(self._modules_dict)

    def keys(self):
        return self._modules_dict.keys()

    def values(self):
        return self._modules_dict.values()

    def items(self):
        return self._modules_dict.items()

"""Thread-local gradient mode. Parity: reference `genesis/grad_mode.py:10-170`.

`no_grad`, `enable_grad` and `set_grad_enabled` work as context managers and as
decorators.
"""
import functools
import threading

_state = threading.local()


def is_grad_enabled():
    return getattr(_state, "enabled", True)


def _set(mode):
    _state.enabled = bool(mode)


class _GradMode:
    _target = True

    def __init__(self, mode=None):
        self.mode = self._target if mode is None else bool(mode)
        self.prev = None

    def __enter__(self):
        self.prev = is_grad_enabled()
        _set(self.mode)
        return self

    def __exit__(self, *exc):
        _set(self.prev)
        return False

    def __call__(self, fn):
        mode = self.mode

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            prev = is_grad_enabled()
            _set(mode)
            try:
                return fn(*args, **kwargs)
            finally:
                _set(prev)
        return wrapper


class no_grad(_GradMode):
    _target = False

    def __init__(self):
        super().__init__(False)


class enable_grad(_GradMode):
    _target = True

    def __init__(self):
        super().__init__(True)


class set_grad_enabled(_GradMode):
    """Sets the mode immediately (function form) and restores it on `__exit__`."""

    def __init__(self, mode):
        super().__init__(mode)
        self.prev = is_grad_enabled()
        _set(self.mode)

    def __enter__(self):
        return self

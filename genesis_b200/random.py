"""Seed management. Parity: reference `genesis/random.py:16-214`.

`Generator` hands one 31-bit seed per random op (`next_seed`), which keys the
Philox counter RNG of the CUDA kernels. CPU random ops draw from torch's global
CPU generator (as the reference's CPU path does); `manual_seed` also seeds that
generator, so one call makes both device paths reproducible.
"""
import threading
import time

import torch


class Generator:
    def __init__(self, device="cpu"):
        self.device = device
        self._lock = threading.Lock()
        self._seed = None
        self._initial_seed = None
        self._counter = 0
        self._set_default_seed()

    def _set_default_seed(self):
        s = int(time.time() * 1000) % (2 ** 31)
        self._seed = s
        self._initial_seed = s
        self._counter = 0

    def manual_seed(self, seed):
        with self._lock:
            self._seed = int(seed) % (2 ** 63)
            self._initial_seed = self._seed
            self._counter = 0
        return self

    def seed(self):
        self._set_default_seed()
        return self._seed

    def initial_seed(self):
        return self._initial_seed

    def get_state(self):
        with self._lock:
            return {"seed": self._seed, "initial_seed": self._initial_seed, "counter": self._counter}

    def set_state(self, state):
        with self._lock:
            self._seed = state["seed"]
            self._initial_seed = state["initial_seed"]
            self._counter = state["counter"]

    def next_seed(self):
        with self._lock:
            s = (self._seed + self._counter) % (2 ** 31)
            self._counter += 1
            return s

    def next_philox(self):
        """(seed, offset) pair for a Philox-keyed kernel: the key is the user seed,
        the offset is the op counter, so streams of different ops never overlap."""
        with self._lock:
            c = self._counter
            self._counter += 1
            return self._seed % (2 ** 63), c


_default_generator = Generator()


def default_generator():
    return _default_generator


def seed():
    s = _default_generator.seed()
    torch.manual_seed(s)
    return s


def manual_seed(seed):
    _default_generator.manual_seed(seed)
    torch.manual_seed(int(seed))
    return _default_generator


def initial_seed():
    return _default_generator.initial_seed()


def get_rng_state():
    st = _default_generator.get_state()
    st["torch_cpu"] = torch.get_rng_state()
    return st


def set_rng_state(state):
    _default_generator.set_state(state)
    if "torch_cpu" in state:
        torch.set_rng_state(state["torch_cpu"])


def get_seed_for_operation():
    return _default_generator.next_seed()


class fork_rng:
    """Context manager that restores the RNG state on exit."""

    def __init__(self, devices=None, enabled=True):
        self.enabled = enabled
        self._saved = None

    def __enter__(self):
        if self.enabled:
            self._saved = get_rng_state()
        return self

    def __exit__(self, *exc):
        if self.enabled and self._saved is not None:
            set_rng_state(self._saved)
        return False

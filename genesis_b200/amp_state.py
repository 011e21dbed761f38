"""Thread-local autocast state shared by `function.py` and `amp/`.

The reference keeps these flags as process-global module attributes
(`genesis/__init__.py:16-18`); here they are thread-local so a data-loader or
watchdog thread can never observe another thread's autocast region.
"""
import threading

import torch


class _AmpState(threading.local):
    def __init__(self):
        self.enabled = False
        self.dtype = torch.float16
        self.cache = {}


amp_state = _AmpState()

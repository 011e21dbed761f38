from .optimizer import Optimizer, SGD, Adam, AdamW
from . import lr_scheduler
from . import adamw  # noqa: E402,F401

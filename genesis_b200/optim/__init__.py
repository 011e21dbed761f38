from .optimizer import Optimizer, SGD, Adam, AdamW
from . import lr_scheduler

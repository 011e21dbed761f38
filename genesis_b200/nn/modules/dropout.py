"""`Dropout`. Parity: reference `genesis/nn/modules/dropout.py:16-22` (keep with probability
1-p, scale by 1/(1-p)); on CUDA the mask comes from the Philox dropout kernel."""
from .. import functional as F
from .module import Module


class Dropout(Module):
    def __init__(self, p=0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return F.dropout(x, self.p, self.training)

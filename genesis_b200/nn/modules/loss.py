"""Loss modules. Parity: reference `genesis/nn/modules/loss.py:11-277`."""
from .. import functional as F
from .module import Module


def _reduce(x, reduction):
    if reduction == "none":
        return x
    if reduction == "sum":
        return F.sum(x)
    if reduction == "mean":
        return F.mean(x)
    raise ValueError(f"Invalid reduction mode: {reduction}")


class CrossEntropyLoss(Module):
    """Softmax cross-entropy on [N, C] logits and integer targets, one fused kernel each way
    (the reference multiplies log-probabilities by a materialised one-hot matrix)."""

    def __init__(self, weight=None, ignore_index=-100, reduction="mean"):
        super().__init__()
        self.weight_ = weight
        self.ignore_index = ignore_index
        self.reduction = reduction

    @property
    def weight(self):
        return self.weight_

    def forward(self, input, target):
        w = None if self.weight_ is None else self.weight_._t
        return F.cross_entropy(input, target, weight=w, ignore_index=self.ignore_index, reduction=self.reduction)


class SoftmaxLoss(Module):
    def forward(self, logits, y):
        return F.cross_entropy(logits, y)


class MSELoss(Module):
    def __init__(self, reduction="mean"):
        super().__init__()
        self.reduction = reduction

    def forward(self, input, target):
        d = input - target
        return _reduce(d * d, self.reduction)


class L1Loss(Module):
    def __init__(self, reduction="mean"):
        super().__init__()
        self.reduction = reduction

    def forward(self, input, target):
        return _reduce(F.abs(input - target), self.reduction)


class BCELoss(Module):
    def __init__(self, weight=None, reduction="mean"):
        super().__init__()
        self.weight_ = weight
        self.reduction = reduction

    def forward(self, input, target):
        eps = 1e-12
        x = F.clamp(input, eps, 1.0 - eps)
        bce = -(target * F.log(x) + (1 - target) * F.log(1 - x))
        if self.weight_ is not None:
            bce = bce * self.weight_
        return _reduce(bce, self.reduction)


class BCEWithLogitsLoss(Module):
    """max(x, 0) - x*y + log(1 + exp(-|x|)), with optional `pos_weight`."""

    def __init__(self, weight=None, reduction="mean", pos_weight=None):
        super().__init__()
        self.weight_ = weight
        self.reduction = reduction
        self.pos_weight = pos_weight

    def forward(self, input, target):
        softplus_neg = F.log(1 + F.exp(-F.abs(input))) + F.relu(-input)   # log(1 + exp(-x))
        if self.pos_weight is not None:
            lw = 1 + (self.pos_weight - 1) * target
            loss = (1 - target) * input + lw * softplus_neg
        else:
            loss = (1 - target) * input + softplus_neg
        if self.weight_ is not None:
            loss = loss * self.weight_
        return _reduce(loss, self.reduction)

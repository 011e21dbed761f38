"""LR schedulers. Parity: reference `genesis/optim/lr_scheduler.py:3-41` (`LambdaLR` does not
apply `lr_lambda(0)` at construction; the first `step()` uses epoch 0) plus the schedulers
its docs describe (`docs/en/training/advanced-features.md:94-136`)."""
import math


class LambdaLR:
    def __init__(self, optimizer, lr_lambda, last_epoch=-1, verbose=False):
        self.optimizer = optimizer
        self.lr_lambda = lr_lambda
        self.base_lrs = optimizer.lr
        self.last_epoch = last_epoch
        self.verbose = verbose

    def _factor(self, epoch):
        return self.lr_lambda(epoch)

    def step(self, epoch=None):
        self.last_epoch = self.last_epoch + 1 if epoch is None else epoch
        self.optimizer.lr = self.base_lrs * self._factor(self.last_epoch)

    def get_last_lr(self):
        return self.optimizer.lr

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k not in ("optimizer", "lr_lambda")}

    def load_state_dict(self, state):
        self.__dict__.update(state)


def get_cosine_schedule_with_warmup(optimizer, num_warmup_steps, num_training_steps, last_epoch=-1):
    def lr_lambda(step):
        if step < num_warmup_steps:
            return step / max(1, num_warmup_steps)
        progress = (step - num_warmup_steps) / max(1, num_training_steps - num_warmup_steps)
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * progress)))
    return LambdaLR(optimizer, lr_lambda, last_epoch)


class StepLR(LambdaLR):
    def __init__(self, optimizer, step_size, gamma=0.1, last_epoch=-1):
        self.step_size, self.gamma = step_size, gamma
        super().__init__(optimizer, None, last_epoch)

    def _factor(self, epoch):
        return self.gamma ** (epoch // self.step_size)


class ExponentialLR(LambdaLR):
    def __init__(self, optimizer, gamma, last_epoch=-1):
        self.gamma = gamma
        super().__init__(optimizer, None, last_epoch)

    def _factor(self, epoch):
        return self.gamma ** epoch


class CosineAnnealingLR(LambdaLR):
    def __init__(self, optimizer, T_max, eta_min=0.0, last_epoch=-1):
        self.T_max, self.eta_min = T_max, eta_min
        super().__init__(optimizer, None, last_epoch)

    def step(self, epoch=None):
        self.last_epoch = self.last_epoch + 1 if epoch is None else epoch
        self.optimizer.lr = self.eta_min + (self.base_lrs - self.eta_min) * \
            (1 + math.cos(math.pi * self.last_epoch / self.T_max)) / 2

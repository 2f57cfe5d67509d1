"""Learning-rate schedules (cells) and ``dynamic_lr`` list builders.
Parity: mindspore/python/mindspore/nn/learning_rate_schedule.py and nn/dynamic_lr.py."""
import math

import torch

from ..ops.primitive import _wrap_out
from .cell import Cell


class LearningRateSchedule(Cell):
    def __init__(self):
        super().__init__()
        self._use_graph = False

    def construct(self, global_step):
        raise NotImplementedError


def _f(step):
    """The step as an fp32 0-d tensor: every schedule below is tensor arithmetic, so a schedule evaluated while a
    graph is traced becomes graph nodes fed by ``global_step`` instead of a constant."""
    if isinstance(step, torch.Tensor):
        return step.detach().as_subclass(torch.Tensor).reshape(()).to(torch.float32)
    return torch.tensor(float(step), dtype=torch.float32)


def _check(lr, rate, steps, name):
    if not isinstance(lr, float) or lr <= 0:
        raise ValueError("For '%s', the 'learning_rate' must be a positive float, but got %r" % (name, lr))
    if rate is not None and (not isinstance(rate, float) or rate <= 0):
        raise ValueError("For '%s', the 'decay_rate' must be a positive float, but got %r" % (name, rate))
    if not isinstance(steps, int) or isinstance(steps, bool) or steps <= 0:
        raise ValueError("For '%s', the 'decay_steps' must be a positive int, but got %r" % (name, steps))


class ExponentialDecayLR(LearningRateSchedule):
    def __init__(self, learning_rate, decay_rate, decay_steps, is_stair=False):
        super().__init__()
        _check(learning_rate, decay_rate, decay_steps, "ExponentialDecayLR")
        self.lr, self.rate, self.steps, self.stair = learning_rate, decay_rate, decay_steps, is_stair

    def construct(self, global_step):
        p = _f(global_step) / self.steps
        if self.stair:
            p = torch.floor(p)
        return _wrap_out(self.lr * torch.pow(torch.tensor(self.rate, dtype=torch.float32), p))


class NaturalExpDecayLR(ExponentialDecayLR):
    def construct(self, global_step):
        p = _f(global_step)
        if self.stair:
            p = torch.floor(p / self.steps) * self.steps
        return _wrap_out(self.lr * torch.exp(-self.rate * p))


class InverseDecayLR(ExponentialDecayLR):
    def construct(self, global_step):
        p = _f(global_step) / self.steps
        if self.stair:
            p = torch.floor(p)
        return _wrap_out(self.lr / (1 + self.rate * p))


class CosineDecayLR(LearningRateSchedule):
    def __init__(self, min_lr, max_lr, decay_steps):
        super().__init__()
        if min_lr >= max_lr:
            raise ValueError("For 'CosineDecayLR', 'max_lr' must be greater than 'min_lr'")
        if not isinstance(decay_steps, int) or decay_steps <= 0:
            raise ValueError("For 'CosineDecayLR', 'decay_steps' must be a positive int")
        self.min_lr, self.max_lr, self.steps = min_lr, max_lr, decay_steps

    def construct(self, global_step):
        p = torch.clamp(_f(global_step), max=float(self.steps))
        return _wrap_out(self.min_lr + 0.5 * (self.max_lr - self.min_lr) * (1 + torch.cos(math.pi * p / self.steps)))


class PolynomialDecayLR(LearningRateSchedule):
    def __init__(self, learning_rate, end_learning_rate, decay_steps, power, update_decay_steps=False):
        super().__init__()
        self.lr, self.end, self.steps, self.power, self.update = learning_rate, end_learning_rate, decay_steps, power, update_decay_steps

    def construct(self, global_step):
        s = _f(global_step)
        steps = torch.tensor(float(self.steps))
        if self.update:
            steps = steps * torch.clamp(torch.ceil(s / steps), min=1.0)
        s = torch.minimum(s, steps)
        return _wrap_out((self.lr - self.end) * torch.pow(1 - s / steps, self.power) + self.end)


class WarmUpLR(LearningRateSchedule):
    def __init__(self, learning_rate, warmup_steps):
        super().__init__()
        if not isinstance(warmup_steps, int) or warmup_steps <= 0:
            raise ValueError("For 'WarmUpLR', 'warmup_steps' must be a positive int")
        self.lr, self.warm = learning_rate, warmup_steps

    def construct(self, global_step):
        return _wrap_out(self.lr * torch.clamp(_f(global_step), max=float(self.warm)) / self.warm)


# ---- list builders (nn/dynamic_lr.py)
def piecewise_constant_lr(milestone, learning_rates):
    if len(milestone) != len(learning_rates):
        raise ValueError("'milestone' and 'learning_rates' must have the same length")
    out, last = [], 0
    for m, lr in zip(milestone, learning_rates):
        if m <= last:
            raise ValueError("'milestone' must be strictly increasing")
        out += [lr] * (m - last)
        last = m
    return out


def exponential_decay_lr(learning_rate, decay_rate, total_step, step_per_epoch, decay_epoch, is_stair=False):
    return [learning_rate * decay_rate ** ((math.floor(math.floor(i / step_per_epoch) / decay_epoch)) if is_stair
                                           else math.floor(i / step_per_epoch) / decay_epoch) for i in range(total_step)]


def natural_exp_decay_lr(learning_rate, decay_rate, total_step, step_per_epoch, decay_epoch, is_stair=False):
    out = []
    for i in range(total_step):
        e = math.floor(i / step_per_epoch)
        if is_stair:
            e = math.floor(e / decay_epoch) * decay_epoch
        out.append(learning_rate * math.exp(-decay_rate * e))
    return out


def inverse_decay_lr(learning_rate, decay_rate, total_step, step_per_epoch, decay_epoch, is_stair=False):
    out = []
    for i in range(total_step):
        e = math.floor(i / step_per_epoch) / decay_epoch
        if is_stair:
            e = math.floor(e)
        out.append(learning_rate / (1 + decay_rate * e))
    return out


def cosine_decay_lr(min_lr, max_lr, total_step, step_per_epoch, decay_epoch):
    return [min_lr + 0.5 * (max_lr - min_lr) * (1 + math.cos(math.pi * min(math.floor(i / step_per_epoch), decay_epoch) / decay_epoch))
            for i in range(total_step)]


def polynomial_decay_lr(learning_rate, end_learning_rate, total_step, step_per_epoch, decay_epoch, power,
                        update_decay_epoch=False):
    out = []
    for i in range(total_step):
        e = math.floor(i / step_per_epoch)
        de = decay_epoch
        if update_decay_epoch:
            de = decay_epoch * max(1, math.ceil(e / decay_epoch))
        e = min(e, de)
        out.append((learning_rate - end_learning_rate) * (1 - e / de) ** power + end_learning_rate)
    return out


def warmup_lr(learning_rate, total_step, step_per_epoch, warmup_epoch):
    return [learning_rate * min(math.floor(i / step_per_epoch), warmup_epoch) / warmup_epoch if warmup_epoch else learning_rate
            for i in range(total_step)]

"""Loss-scale managers.  Parity: mindspore/python/mindspore/train/loss_scale_manager.py:48,121."""
from ..nn import wrap


class LossScaleManager:
    def get_loss_scale(self): pass
    def update_loss_scale(self, overflow): pass
    def get_update_cell(self): pass


class FixedLossScaleManager(LossScaleManager):
    def __init__(self, loss_scale=128.0, drop_overflow_update=True):
        if loss_scale < 1:
            raise ValueError("The argument 'loss_scale' must be >= 1, but got %s" % loss_scale)
        self._loss_scale = loss_scale
        self._drop_overflow_update = drop_overflow_update

    def get_loss_scale(self):
        return self._loss_scale

    def get_drop_overflow_update(self):
        return self._drop_overflow_update

    def update_loss_scale(self, overflow):
        pass

    def get_update_cell(self):
        if not self._drop_overflow_update:
            return None
        return wrap.FixedLossScaleUpdateCell(self._loss_scale)


class DynamicLossScaleManager(LossScaleManager):
    def __init__(self, init_loss_scale=2 ** 24, scale_factor=2, scale_window=2000):
        if init_loss_scale < 1.0:
            raise ValueError("The argument 'init_loss_scale' must be >= 1, but got %s" % init_loss_scale)
        if scale_factor <= 0:
            raise ValueError("The argument 'scale_factor' must be > 0, but got %s" % scale_factor)
        if scale_window <= 0:
            raise ValueError("The argument 'scale_window' must be > 0, but got %s" % scale_window)
        self.loss_scale, self.scale_factor, self.scale_window = init_loss_scale, scale_factor, scale_window
        self.cur_iter, self.last_overflow_iter = 1, 0
        self.increase_ratio, self.decrease_ratio = scale_factor, 1 / scale_factor

    def get_loss_scale(self):
        return self.loss_scale

    def update_loss_scale(self, overflow):
        if overflow:
            self.loss_scale = max(self.loss_scale * self.decrease_ratio, 1)
            self.last_overflow_iter = self.cur_iter
        elif (self.cur_iter - self.last_overflow_iter) % self.scale_window == 0:
            self.loss_scale *= self.increase_ratio
        self.cur_iter += 1

    def get_drop_overflow_update(self):
        return True

    def get_update_cell(self):
        return wrap.DynamicLossScaleUpdateCell(self.loss_scale, self.scale_factor, self.scale_window)

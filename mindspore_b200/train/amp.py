"""Automatic mixed precision.

Levels: O0 fp32; O1 cast the white-list cells (Conv*, Dense, matmul-like) to the low-precision dtype;
O2/O3 cast the whole network except (O2) normalisation layers; "auto" = O2 on GPU.  The low-precision dtype
is bf16 on this runtime (fp16 can be requested with ``dtype=``).  ``build_train_network`` then wraps loss,
optional loss scaling and the step cell like the reference.

Parity: mindspore/python/mindspore/train/amp.py:305-404 (auto_mixed_precision), :485 (_add_loss_network),
:542-647 (build_train_network); mindspore/python/mindspore/amp.py (DynamicLossScaler, StaticLossScaler,
all_finite).
"""
import torch

from .. import context
from ..common import dtype as mstype
from ..nn import layer as L
from ..nn import wrap
from ..nn.cell import Cell
from ..ops.primitive import _wrap_out

AMP_WHITE_LIST = [L.Conv1d, L.Conv2d, L.Conv2dTranspose, L.Dense, L.LSTM, L.GRU, L.RNN]
AMP_BLACK_LIST = [L.BatchNorm1d, L.BatchNorm2d, L.BatchNorm3d, L.LayerNorm, L.SyncBatchNorm, L.GroupNorm]


def get_white_list():
    return list(AMP_WHITE_LIST)


def get_black_list():
    return list(AMP_BLACK_LIST)


class _OutputTo32(Cell):
    def __init__(self, backbone):
        super().__init__(auto_prefix=False)
        self._backbone = backbone

    def construct(self, *args):
        out = self._backbone(*args)
        if isinstance(out, torch.Tensor) and out.is_floating_point():
            return out.float()
        if isinstance(out, (tuple, list)):
            return type(out)(o.float() if isinstance(o, torch.Tensor) and o.is_floating_point() else o for o in out)
        return out


class _OutputTo16(Cell):
    def __init__(self, backbone, dtype=mstype.bfloat16):
        super().__init__(auto_prefix=False)
        self._backbone, self.dtype = backbone, dtype

    def construct(self, *args):
        return self._backbone(*args).to(self.dtype)


def auto_mixed_precision(network, amp_level="O0", dtype=mstype.bfloat16, custom_white_list=None,
                         custom_black_list=None):
    if not isinstance(network, Cell):
        raise TypeError("The network type should be Cell.")
    if amp_level == "auto":
        amp_level = "O2" if context.get_context("device_target") == "GPU" else "O0"
    if amp_level not in ("O0", "O1", "O2", "O3"):
        raise ValueError("The amp level %r is not supported" % amp_level)
    if dtype not in (mstype.float16, mstype.bfloat16):
        raise ValueError("The dtype should be one of (float16, bfloat16), but got %s" % dtype)
    if amp_level == "O0":
        return network
    white = tuple(custom_white_list or AMP_WHITE_LIST)
    black = tuple(custom_black_list or AMP_BLACK_LIST)
    if amp_level == "O1":
        for _, c in network.cells_and_names():
            if isinstance(c, white):
                c.to_float(dtype)
    elif amp_level == "O2":
        network.to_float(dtype)
        for _, c in network.cells_and_names():
            if isinstance(c, black):
                c.to_float(mstype.float32)
    else:
        network.to_float(dtype)
    network._mixed_precision_type = dtype
    return network


def _add_loss_network(network, loss_fn, cast_model_type):
    class WithLossCell(Cell):
        def __init__(self, backbone, loss_fn):
            super().__init__(auto_prefix=False)
            self._backbone, self._loss_fn = backbone, loss_fn

        def construct(self, data, label):
            out = self._backbone(data)
            if isinstance(out, torch.Tensor) and out.dtype != torch.float32 and not out.is_cuda:
                out = out.float()
            return self._loss_fn(out, label)

    if cast_model_type in (mstype.float16, mstype.bfloat16):
        return WithLossCell(network, loss_fn)
    return wrap.WithLossCell(network, loss_fn)


def build_train_network(network, optimizer, loss_fn=None, level="O0", boost_level="O0", **kwargs):
    if level not in ("O0", "O1", "O2", "O3", "auto"):
        raise ValueError("level must be one of O0, O1, O2, O3, auto")
    if level == "auto":
        level = "O2" if context.get_context("device_target") == "GPU" else "O0"
    cast_type = kwargs.get("cast_model_type", mstype.float32 if level == "O0" else mstype.bfloat16)
    loss_scale_manager = kwargs.get("loss_scale_manager")
    if level != "O0":
        auto_mixed_precision(network, level, cast_type if cast_type != mstype.float32 else mstype.bfloat16)
    if loss_fn is not None:
        network = _add_loss_network(network, loss_fn, cast_type)
    stages = context.get_auto_parallel_context("pipeline_stages")
    accu = context.get_auto_parallel_context("grad_accumulation_step")
    if loss_scale_manager is not None:
        update_cell = loss_scale_manager.get_update_cell()
        if update_cell is not None:
            return wrap.TrainOneStepWithLossScaleCell(network, optimizer, scale_sense=update_cell).set_train()
        sens = loss_scale_manager.get_loss_scale()
        cls = wrap._TrainGradAccuStepCell if (stages > 1 or accu > 1) else wrap.TrainOneStepCell
        return cls(network, optimizer, sens).set_train()
    cls = wrap._TrainGradAccuStepCell if (stages > 1 or accu > 1) else wrap.TrainOneStepCell
    return cls(network, optimizer).set_train()


# ---- functional loss scalers (mindspore.amp)
def all_finite(inputs):
    ok = None
    for x in (inputs if isinstance(inputs, (tuple, list)) else [inputs]):
        f = torch.isfinite(x).all()
        ok = f if ok is None else ok & f
    return _wrap_out(ok)


class LossScaler:
    def scale(self, inputs): raise NotImplementedError
    def unscale(self, inputs): raise NotImplementedError
    def adjust(self, grads_finite): raise NotImplementedError


class StaticLossScaler(LossScaler):
    def __init__(self, scale_value):
        if scale_value < 1.0:
            raise ValueError("The argument 'scale_value' must be > 1, but got %s" % scale_value)
        self.scale_value = float(scale_value)

    def scale(self, inputs):
        return _map(inputs, lambda x: x * self.scale_value)

    def unscale(self, inputs):
        return _map(inputs, lambda x: x / self.scale_value)

    def adjust(self, grads_finite):
        return False


class DynamicLossScaler(LossScaler):
    def __init__(self, scale_value, scale_factor, scale_window):
        if scale_value < 1.0:
            raise ValueError("The argument 'scale_value' must be > 1, but got %s" % scale_value)
        self.scale_value, self.scale_factor, self.scale_window = float(scale_value), scale_factor, scale_window
        self.counter = 0

    def scale(self, inputs):
        return _map(inputs, lambda x: x * self.scale_value)

    def unscale(self, inputs):
        return _map(inputs, lambda x: x / self.scale_value)

    def adjust(self, grads_finite):
        if bool(grads_finite):
            self.counter += 1
            if self.counter >= self.scale_window:
                self.scale_value *= self.scale_factor
                self.counter = 0
        else:
            self.scale_value = max(1.0, self.scale_value / self.scale_factor)
            self.counter = 0
        return True


def _map(x, fn):
    if isinstance(x, (tuple, list)):
        return type(x)(_map(v, fn) for v in x)
    return _wrap_out(fn(x))


def custom_mixed_precision(network, *, white_list=None, black_list=None, dtype=mstype.float16):
    """Casts by an explicit list: with ``white_list`` only cells (or primitives' owning cells) of those types run in
    ``dtype``; with ``black_list`` everything runs in ``dtype`` except those types.  Exactly one list must be given."""
    if not isinstance(network, Cell):
        raise TypeError("The network type should be Cell.")
    if (white_list is None) == (black_list is None):
        raise ValueError("For custom_mixed_precision, exactly one of white_list and black_list must be given")
    if dtype not in (mstype.float16, mstype.bfloat16):
        raise ValueError("The dtype should be one of (float16, bfloat16), but got %s" % dtype)
    if white_list is not None:
        kinds = tuple(t for t in white_list if isinstance(t, type))
        for _, c in network.cells_and_names():
            if kinds and isinstance(c, kinds):
                c.to_float(dtype)
    else:
        kinds = tuple(t for t in black_list if isinstance(t, type))
        network.to_float(dtype)
        for _, c in network.cells_and_names():
            if kinds and isinstance(c, kinds):
                c.to_float(mstype.float32)
    network._mixed_precision_type = dtype
    return network


def init_status():
    """Fresh overflow-status tensor (eight zeros); the overflow check itself is ``all_finite`` on the gradients."""
    import torch
    from ..common.tensor import Tensor
    return Tensor(torch.zeros(8, dtype=torch.float32))

from .loss_scale_manager import DynamicLossScaleManager, FixedLossScaleManager, LossScaleManager  # noqa: E402,F401

"""``Model``: high-level train / eval / predict driver.

Parity: mindspore/python/mindspore/train/model.py:258 (ctor), :445-475 (_build_train_network), :750-816
(_train), :822-949 (sink loop), :1066 (non-sink loop), :1178 (train), :1424 (fit), :1631 (eval), :1796
(predict), :1998 (infer_train_layout), :2066 (infer_predict_layout).  "Sink" mode here means the host
prefetches and copies the next batch (pinned memory -> device on a side stream) while the current step runs.
"""
from __future__ import annotations

import os

import torch

from .. import context
from ..common.tensor import Tensor
from ..nn.cell import Cell
from ..nn import wrap
from ..nn.optim import Optimizer
from . import amp as _amp
from .callback import CallbackManager, RunContext, _InternalCallbackParam
from .dataset_helper import DatasetHelper
from .loss_scale_manager import LossScaleManager
from .metrics import get_metrics


def _to_device(x, dev):
    if isinstance(x, torch.Tensor):
        if x.device != dev:
            x = x.to(dev, non_blocking=True)
        return x if isinstance(x, Tensor) else x.as_subclass(Tensor)
    if isinstance(x, (list, tuple)):
        return type(x)(_to_device(v, dev) for v in x)
    try:
        import numpy as np
        if isinstance(x, np.ndarray):
            return Tensor(x)
    except ImportError:
        pass
    return x


class Model:
    def __init__(self, network, loss_fn=None, optimizer=None, metrics=None, eval_network=None, eval_indexes=None,
                 amp_level="O0", boost_level="O0", **kwargs):
        if not isinstance(network, Cell):
            raise TypeError("For 'Model', the argument 'network' must be a Cell, but got %s" % type(network))
        if amp_level not in ("O0", "O1", "O2", "O3", "auto"):
            raise ValueError("For 'Model', 'amp_level' must be one of O0, O1, O2, O3, auto, but got %r" % amp_level)
        for k in kwargs:
            if k not in ("loss_scale_manager", "keep_batchnorm_fp32"):
                raise ValueError("The argument %r is not supported by Model" % k)
        if optimizer is not None and not isinstance(optimizer, Optimizer):
            raise TypeError("For 'Model', the argument 'optimizer' must be an Optimizer")
        if eval_indexes is not None and (not isinstance(eval_indexes, list) or len(eval_indexes) != 3):
            raise ValueError("The argument 'eval_indexes' must be a list of 3 ints")
        self._network, self._loss_fn, self._optimizer = network, loss_fn, optimizer
        self._amp_level, self._boost_level = amp_level, boost_level
        self._loss_scale_manager = kwargs.get("loss_scale_manager")
        if self._loss_scale_manager is not None and not isinstance(self._loss_scale_manager, LossScaleManager):
            raise TypeError("'loss_scale_manager' must be a LossScaleManager")
        self._keep_bn_fp32 = kwargs.get("keep_batchnorm_fp32", True)
        self._metrics = metrics
        self._metric_fns = get_metrics(metrics) if metrics else {}
        self._eval_network, self._eval_indexes = eval_network, eval_indexes
        self._parallel_mode = context.get_auto_parallel_context("parallel_mode")
        self._train_network = self._build_train_network()
        self._build_eval_network()
        self._predict_network = None
        self._current_epoch_num = 0
        self._current_step_num = 0
        self.need_load_ckpt = False

    # ------------------------------------------------------------------ network builders
    def _build_train_network(self):
        net = self._network
        if self._optimizer is not None:
            net = _amp.build_train_network(net, self._optimizer, self._loss_fn, self._amp_level, self._boost_level,
                                           loss_scale_manager=self._loss_scale_manager,
                                           keep_batchnorm_fp32=self._keep_bn_fp32)
        elif self._loss_fn is not None:
            net = wrap.WithLossCell(net, self._loss_fn)
        return net

    def _build_eval_network(self):
        if not self._metric_fns:
            return
        if self._eval_network is None:
            if self._loss_fn is None:
                raise ValueError("If 'metrics' is set, 'loss_fn' or 'eval_network' must be set too")
            self._eval_network = wrap.WithEvalCell(self._network, self._loss_fn,
                                                   self._amp_level in ("O2", "O3", "auto"))
            self._eval_indexes = [0, 1, 2]

    @property
    def train_network(self):
        return self._train_network

    @property
    def predict_network(self):
        return self._predict_network or self._network

    @property
    def eval_network(self):
        return self._eval_network

    def build(self, train_dataset=None, valid_dataset=None, sink_size=-1, epoch=1):
        """Pre-compiles the graphs when running in GRAPH mode (first batch shapes)."""
        if train_dataset is not None and context.get_context("mode") == context.GRAPH_MODE:
            it = iter(DatasetHelper(train_dataset, False))
            try:
                batch = next(it)
            except StopIteration:
                return
            self._train_network.compile(*_to_device(tuple(batch), context.device()))

    # ------------------------------------------------------------------ training
    def _callback_param(self, epoch, ds_size, mode="train"):
        p = _InternalCallbackParam()
        p.train_network = self._train_network
        p.network = self._network
        p.epoch_num = epoch
        p.batch_num = ds_size
        p.mode = mode
        p.loss_fn = self._loss_fn
        p.optimizer = self._optimizer
        p.parallel_mode = self._parallel_mode
        p.cur_step_num = 0
        p.cur_epoch_num = 0
        p.metrics = None
        p.eval_results = None
        return p

    def train(self, epoch, train_dataset, callbacks=None, dataset_sink_mode=False, sink_size=-1, initial_epoch=0):
        if not isinstance(epoch, int) or epoch <= 0:
            raise ValueError("For 'Model.train', 'epoch' must be a positive int, but got %r" % (epoch,))
        if initial_epoch < 0 or initial_epoch >= epoch:
            raise ValueError("For 'Model.train', 'initial_epoch' must be in [0, epoch)")
        if self._optimizer is None and self._loss_fn is None and not isinstance(self._network, wrap.TrainOneStepCell):
            pass
        self._train(epoch, train_dataset, callbacks, dataset_sink_mode, sink_size, initial_epoch)

    def _train(self, epoch, train_dataset, callbacks, sink, sink_size, initial_epoch, valid_dataset=None,
               valid_frequency=1, valid_sink=False):
        helper = DatasetHelper(train_dataset, sink, sink_size)
        ds_size = helper.dataset_size()
        cb = CallbackManager(callbacks)
        p = self._callback_param(epoch, ds_size)
        rc = RunContext(p)
        net = self._train_network
        net.set_train(True)
        dev = context.device()
        self._check_recovery(p)
        cb.on_train_begin(rc)
        start_epoch = max(initial_epoch, p.get("restored_epoch", 0) or 0)
        p.cur_step_num = start_epoch * ds_size
        for ep in range(start_epoch, epoch):
            p.cur_epoch_num = ep + 1
            cb.on_train_epoch_begin(rc)
            for batch in helper:
                p.cur_step_num += 1
                inputs = _to_device(tuple(batch) if isinstance(batch, (tuple, list)) else (batch,), dev)
                p.train_dataset_element = inputs
                cb.on_train_step_begin(rc)
                p.net_outputs = net(*inputs)
                cb.on_train_step_end(rc)
                if rc.get_stop_requested():
                    break
            if valid_dataset is not None and (ep + 1) % valid_frequency == 0:
                p.eval_results = self.eval(valid_dataset, dataset_sink_mode=valid_sink)
                p.metrics = p.eval_results
                net.set_train(True)
            cb.on_train_epoch_end(rc)
            if rc.get_stop_requested():
                break
        cb.on_train_end(rc)
        self._current_epoch_num, self._current_step_num = p.cur_epoch_num, p.cur_step_num

    def _check_recovery(self, p):
        """MS_ENABLE_RECOVERY: reload the latest checkpoint every rank has (reference model.py:991-1064)."""
        from ..parallel.recovery import recovery_context
        rcx = recovery_context()
        if not rcx.enabled:
            return
        info = rcx.latest_common_checkpoint()
        if info is not None:
            from .serialization import load_checkpoint, load_param_into_net
            d = load_checkpoint(info["path"])
            load_param_into_net(self._train_network, d)
            p.restored_epoch = info["epoch"]

    def fit(self, epoch, train_dataset, valid_dataset=None, valid_frequency=1, callbacks=None,
            dataset_sink_mode=False, valid_dataset_sink_mode=False, sink_size=-1, initial_epoch=0):
        if valid_dataset is not None and not self._metric_fns:
            raise ValueError("For 'Model.fit', if valid_dataset is not None, the model argument 'metrics' can not "
                             "be None or empty")
        self._train(epoch, train_dataset, callbacks, dataset_sink_mode, sink_size, initial_epoch, valid_dataset,
                    valid_frequency, valid_dataset_sink_mode)

    # ------------------------------------------------------------------ eval / predict
    def eval(self, valid_dataset, callbacks=None, dataset_sink_mode=False):
        if not self._metric_fns:
            raise ValueError("For Model.eval, the model argument 'metrics' can not be None or empty, you should "
                             "set the argument 'metrics' for model.")
        net = self._eval_network
        net.set_train(False)
        for m in self._metric_fns.values():
            m.clear()
        helper = DatasetHelper(valid_dataset, dataset_sink_mode)
        cb = CallbackManager(callbacks)
        p = self._callback_param(1, helper.dataset_size(), "eval")
        rc = RunContext(p)
        cb.on_eval_begin(rc)
        cb.on_eval_epoch_begin(rc)
        dev = context.device()
        with torch.no_grad():
            for batch in helper:
                p.cur_step_num += 1
                cb.on_eval_step_begin(rc)
                outputs = net(*_to_device(tuple(batch), dev))
                p.net_outputs = outputs
                self._update_metrics(outputs)
                cb.on_eval_step_end(rc)
                if rc.get_stop_requested():
                    break
        cb.on_eval_epoch_end(rc)
        res = {k: m.eval() for k, m in self._metric_fns.items()}
        p.metrics = res
        cb.on_eval_end(rc)
        return res

    def _update_metrics(self, outputs):
        if not isinstance(outputs, (tuple, list)):
            raise ValueError("The 'outputs' of the eval network should be tuple or list")
        idx = self._eval_indexes
        for m in self._metric_fns.values():
            if m.__class__.__name__ == "Loss":
                m.update(outputs[idx[0]] if idx else outputs[0])
            else:
                m.update(*(outputs[idx[1]], outputs[idx[2]]) if idx else outputs)

    def predict(self, *predict_data, backend=None, config=None):
        net = self._predict_network or self._network
        net.set_train(False)
        with torch.no_grad():
            return net(*_to_device(predict_data, context.device()))

    # ------------------------------------------------------------------ layouts
    def infer_train_layout(self, train_dataset, dataset_sink_mode=True, sink_size=-1):
        self.build(train_dataset)
        return self._train_network.parameter_layout_dict

    def infer_predict_layout(self, *predict_data, skip_backend_compile=False):
        net = self._predict_network or self._network
        if context.get_context("mode") == context.GRAPH_MODE:
            net.compile(*predict_data)
        return net.parameter_layout_dict

"""Training callbacks.

Parity: mindspore/python/mindspore/train/callback/_callback.py (Callback, RunContext, CallbackManager,
_InternalCallbackParam), _checkpoint.py:101 (CheckpointConfig), :412 (ModelCheckpoint), _loss_monitor.py,
_time_monitor.py, _early_stop.py, _reduce_lr_on_plateau.py, _lr_scheduler_callback.py, _history.py,
_lambda_callback.py, _backup_and_restore.py, _on_request_exit.py, _flops_collector.py, _cluster_monitor.py.
"""
from __future__ import annotations

import json
import os
import signal
import time

import numpy as np
import torch

from ..utils.log import logger


class _InternalCallbackParam(dict):
    def __getattr__(self, k):
        return self.get(k)

    def __setattr__(self, k, v):
        self[k] = v


class RunContext:
    def __init__(self, original_args):
        if not isinstance(original_args, dict):
            raise TypeError("The argument 'original_args' of RunContext should be dict type")
        self._original_args = original_args
        self._stop_requested = False

    def original_args(self):
        return self._original_args

    def request_stop(self):
        self._stop_requested = True

    def get_stop_requested(self):
        return self._stop_requested


class Callback:
    def __enter__(self):
        return self

    def __exit__(self, *err):
        pass

    def begin(self, run_context): pass
    def epoch_begin(self, run_context): pass
    def epoch_end(self, run_context): pass
    def step_begin(self, run_context): pass
    def step_end(self, run_context): pass
    def end(self, run_context): pass

    def on_train_begin(self, run_context): self.begin(run_context)
    def on_train_epoch_begin(self, run_context): self.epoch_begin(run_context)
    def on_train_epoch_end(self, run_context): self.epoch_end(run_context)
    def on_train_step_begin(self, run_context): self.step_begin(run_context)
    def on_train_step_end(self, run_context): self.step_end(run_context)
    def on_train_end(self, run_context): self.end(run_context)
    def on_eval_begin(self, run_context): pass
    def on_eval_epoch_begin(self, run_context): pass
    def on_eval_epoch_end(self, run_context): pass
    def on_eval_step_begin(self, run_context): pass
    def on_eval_step_end(self, run_context): pass
    def on_eval_end(self, run_context): pass


class CallbackManager(Callback):
    def __init__(self, callbacks):
        self._callbacks = []
        if callbacks is None:
            return
        if isinstance(callbacks, Callback):
            callbacks = [callbacks]
        for cb in callbacks:
            if not isinstance(cb, Callback):
                raise TypeError("When the 'callbacks' is a list, the elements in 'callbacks' must be Callback "
                                "functions.")
            self._callbacks.append(cb)

    def _all(self, name, rc):
        for cb in self._callbacks:
            getattr(cb, name)(rc)

    def on_train_begin(self, rc): self._all("on_train_begin", rc)
    def on_train_epoch_begin(self, rc): self._all("on_train_epoch_begin", rc)
    def on_train_epoch_end(self, rc): self._all("on_train_epoch_end", rc)
    def on_train_step_begin(self, rc): self._all("on_train_step_begin", rc)
    def on_train_step_end(self, rc): self._all("on_train_step_end", rc)
    def on_train_end(self, rc): self._all("on_train_end", rc)
    def on_eval_begin(self, rc): self._all("on_eval_begin", rc)
    def on_eval_epoch_begin(self, rc): self._all("on_eval_epoch_begin", rc)
    def on_eval_epoch_end(self, rc): self._all("on_eval_epoch_end", rc)
    def on_eval_step_begin(self, rc): self._all("on_eval_step_begin", rc)
    def on_eval_step_end(self, rc): self._all("on_eval_step_end", rc)
    def on_eval_end(self, rc): self._all("on_eval_end", rc)


def _loss_value(out):
    if isinstance(out, (tuple, list)):
        out = out[0]
    if isinstance(out, torch.Tensor):
        return float(out.detach().float().mean())
    return float(out)


class LossMonitor(Callback):
    def __init__(self, per_print_times=1):
        if not isinstance(per_print_times, int) or per_print_times < 0:
            raise ValueError("The argument 'per_print_times' must be int and >= 0, but got %r" % (per_print_times,))
        self._per_print_times = per_print_times
        self.losses = []

    def on_train_step_end(self, run_context):
        p = run_context.original_args()
        loss = _loss_value(p.net_outputs)
        self.losses.append(loss)
        if np.isnan(loss) or np.isinf(loss):
            raise ValueError("epoch: %d step: %d. Invalid loss, terminating training." % (p.cur_epoch_num,
                                                                                          p.cur_step_num))
        if self._per_print_times and p.cur_step_num % self._per_print_times == 0:
            step_in_epoch = (p.cur_step_num - 1) % p.batch_num + 1
            print("epoch: %d step: %d, loss is %s" % (p.cur_epoch_num, step_in_epoch, loss), flush=True)


class TimeMonitor(Callback):
    def __init__(self, data_size=None, data_time=False):
        self.data_size = data_size
        self.epoch_time = None
        self.step_times = []

    def on_train_epoch_begin(self, run_context):
        self.epoch_time = time.time()

    def on_train_step_begin(self, run_context):
        self._t = time.time()

    def on_train_step_end(self, run_context):
        self.step_times.append((time.time() - self._t) * 1000)

    def on_train_epoch_end(self, run_context):
        p = run_context.original_args()
        ms = (time.time() - self.epoch_time) * 1000
        n = self.data_size or p.batch_num
        print("Train epoch time: %5.3f ms, per step time: %5.3f ms" % (ms, ms / max(n, 1)), flush=True)


class History(Callback):
    def begin(self, run_context):
        self.epoch = []
        self.history = {}

    def epoch_end(self, run_context):
        p = run_context.original_args()
        self.epoch.append(p.cur_epoch_num)
        self.history.setdefault("net_output", []).append(_loss_value(p.net_outputs))
        for k, v in (p.metrics or {}).items():
            self.history.setdefault(k, []).append(v)


class LambdaCallback(Callback):
    def __init__(self, on_train_epoch_begin=None, on_train_epoch_end=None, on_train_step_begin=None,
                 on_train_step_end=None, on_train_begin=None, on_train_end=None, on_eval_epoch_begin=None,
                 on_eval_epoch_end=None, on_eval_step_begin=None, on_eval_step_end=None, on_eval_begin=None,
                 on_eval_end=None):
        for k, v in list(locals().items()):
            if k != "self" and v is not None:
                setattr(self, k, v)


class LearningRateScheduler(Callback):
    def __init__(self, learning_rate_function):
        self.fn = learning_rate_function

    def on_train_step_end(self, run_context):
        p = run_context.original_args()
        opt = p.optimizer
        if opt is None:
            return
        old = float(opt.get_lr()) if not opt.is_group_lr else None
        new = self.fn(old, p.cur_step_num)
        if old is None or abs(new - old) > 1e-12:
            opt.learning_rate = float(new)


class EarlyStopping(Callback):
    def __init__(self, monitor="eval_loss", min_delta=0, patience=0, verbose=False, mode="auto", baseline=None,
                 restore_best_weights=False):
        if mode not in ("auto", "min", "max"):
            raise ValueError("mode must be auto, min or max")
        self.monitor, self.min_delta, self.patience, self.baseline = monitor, abs(min_delta), patience, baseline
        self.mode = mode
        self.restore_best_weights = restore_best_weights
        self.wait, self.stopped_epoch, self.best, self.best_weights = 0, 0, None, None

    def _better(self, cur, best):
        maximize = self.mode == "max" or (self.mode == "auto" and ("acc" in self.monitor or "f1" in self.monitor))
        return cur - self.min_delta > best if maximize else cur + self.min_delta < best

    def _value(self, p):
        if self.monitor == "loss":
            return _loss_value(p.net_outputs)
        m = p.eval_results or p.metrics or {}
        return m.get(self.monitor)

    def on_train_begin(self, run_context):
        self.wait, self.stopped_epoch = 0, 0
        self.best = self.baseline

    def on_train_epoch_end(self, run_context):
        p = run_context.original_args()
        cur = self._value(p)
        if cur is None:
            return
        if self.best is None or self._better(cur, self.best):
            self.best, self.wait = cur, 0
            if self.restore_best_weights:
                self.best_weights = {q.name: q.detach().clone() for q in p.train_network.get_parameters()}
        else:
            self.wait += 1
            if self.wait >= self.patience:
                self.stopped_epoch = p.cur_epoch_num
                run_context.request_stop()
                if self.restore_best_weights and self.best_weights:
                    for q in p.train_network.get_parameters():
                        q.set_data(self.best_weights[q.name])


class ReduceLROnPlateau(Callback):
    def __init__(self, monitor="eval_loss", factor=0.1, patience=10, verbose=False, mode="auto", min_delta=1e-4,
                 cooldown=0, min_lr=0):
        if factor >= 1.0:
            raise ValueError("The learning rate reduction factor should be less than 1.0")
        self.monitor, self.factor, self.patience, self.mode = monitor, factor, patience, mode
        self.min_delta, self.cooldown, self.min_lr = min_delta, cooldown, min_lr
        self.wait, self.cooldown_counter, self.best = 0, 0, None

    def on_train_epoch_end(self, run_context):
        p = run_context.original_args()
        cur = _loss_value(p.net_outputs) if self.monitor == "loss" else (p.eval_results or p.metrics or {}).get(self.monitor)
        if cur is None:
            return
        if self.cooldown_counter > 0:
            self.cooldown_counter -= 1
            self.wait = 0
        better = self.best is None or (cur > self.best + self.min_delta if self.mode == "max"
                                       else cur < self.best - self.min_delta)
        if better:
            self.best, self.wait = cur, 0
        elif self.cooldown_counter <= 0:
            self.wait += 1
            if self.wait >= self.patience:
                opt = p.optimizer
                old = float(opt.get_lr())
                opt.learning_rate = max(old * self.factor, self.min_lr)
                self.cooldown_counter, self.wait = self.cooldown, 0


class CheckpointConfig:
    def __init__(self, save_checkpoint_steps=1, save_checkpoint_seconds=0, keep_checkpoint_max=5,
                 keep_checkpoint_per_n_minutes=0, integrated_save=True, async_save=False, saved_network=None,
                 append_info=None, enc_key=None, enc_mode="AES-GCM", exception_save=False, crc_check=False,
                 remove_redundancy=False, **kwargs):
        for n, v in (("save_checkpoint_steps", save_checkpoint_steps), ("save_checkpoint_seconds", save_checkpoint_seconds),
                     ("keep_checkpoint_max", keep_checkpoint_max), ("keep_checkpoint_per_n_minutes", keep_checkpoint_per_n_minutes)):
            if v is not None and (not isinstance(v, int) or isinstance(v, bool) or v < 0):
                raise ValueError("For 'CheckpointConfig', '%s' must be a non-negative int, but got %r" % (n, v))
        if not save_checkpoint_steps and not save_checkpoint_seconds and not keep_checkpoint_max and \
                not keep_checkpoint_per_n_minutes:
            raise ValueError("For 'CheckpointConfig', the input arguments can't all be None or 0")
        self.save_checkpoint_steps = save_checkpoint_steps
        self.save_checkpoint_seconds = save_checkpoint_seconds
        if save_checkpoint_steps and save_checkpoint_seconds:
            self.save_checkpoint_seconds = 0
        self.keep_checkpoint_max = keep_checkpoint_max
        self.keep_checkpoint_per_n_minutes = keep_checkpoint_per_n_minutes
        if keep_checkpoint_max and keep_checkpoint_per_n_minutes:
            self.keep_checkpoint_per_n_minutes = 0
        self.integrated_save, self.async_save, self.saved_network = integrated_save, async_save, saved_network
        self.append_dict = self._handle_append_info(append_info)
        self.enc_key, self.enc_mode, self.exception_save, self.crc_check = enc_key, enc_mode, exception_save, crc_check
        self.remove_redundancy = remove_redundancy

    @staticmethod
    def _handle_append_info(append_info):
        if append_info is None:
            return None
        if not isinstance(append_info, list):
            raise TypeError("The type of 'append_info' must be list, but got %s" % type(append_info))
        out = {}
        for el in append_info:
            if isinstance(el, str):
                if el not in ("epoch_num", "step_num"):
                    raise TypeError("The str element of 'append_info' must be 'epoch_num' or 'step_num'")
                out[el] = 0
            elif isinstance(el, dict):
                for k, v in el.items():
                    if not isinstance(k, str) or not isinstance(v, (int, float, bool, str, torch.Tensor)):
                        raise TypeError("The key of append_info dict must be str and the value int/float/bool/str/"
                                        "Tensor")
                    out[k] = v
            else:
                raise TypeError("The element of 'append_info' must be str or dict")
        return out

    def get_checkpoint_policy(self):
        return {k: getattr(self, k) for k in ("save_checkpoint_steps", "save_checkpoint_seconds",
                                              "keep_checkpoint_max", "keep_checkpoint_per_n_minutes", "saved_network")}


class ModelCheckpoint(Callback):
    def __init__(self, prefix="CKP", directory=None, config=None):
        if not isinstance(prefix, str) or "/" in prefix:
            raise ValueError("For 'ModelCheckpoint', the argument 'prefix' for checkpoint file name is invalid, it "
                             "must be string and does not contain '/', but got %r" % (prefix,))
        self._prefix = prefix
        self._directory = os.path.abspath(directory) if directory else os.getcwd()
        os.makedirs(self._directory, exist_ok=True)
        if config is not None and not isinstance(config, CheckpointConfig):
            raise TypeError("For 'ModelCheckpoint', the type of argument 'config' should be 'CheckpointConfig'")
        self._config = config or CheckpointConfig()
        self._last_time = time.time()
        self._last_triggered_step = 0
        self._files = []
        self._latest = ""

    @property
    def latest_ckpt_file_name(self):
        return self._latest

    def _save(self, p, force=False):
        from .serialization import save_checkpoint
        cfg = self._config
        step = p.cur_step_num
        due = force
        if cfg.save_checkpoint_steps and step >= self._last_triggered_step + cfg.save_checkpoint_steps:
            due = True
        if cfg.save_checkpoint_seconds and time.time() - self._last_time >= cfg.save_checkpoint_seconds:
            due = True
        if not due or step == self._last_triggered_step:
            return
        self._last_triggered_step, self._last_time = step, time.time()
        step_in_epoch = (step - 1) % p.batch_num + 1
        from .. import context
        rank_tag = ""
        name = "%s%s-%d_%d.ckpt" % (self._prefix, rank_tag, p.cur_epoch_num, step_in_epoch)
        path = os.path.join(self._directory, name)
        net = cfg.saved_network or p.train_network
        append = dict(cfg.append_dict) if cfg.append_dict else None
        if append is not None:
            if "epoch_num" in append:
                append["epoch_num"] = p.cur_epoch_num
            if "step_num" in append:
                append["step_num"] = step
        mode = context.get_auto_parallel_context("parallel_mode")
        integrated = cfg.integrated_save and mode in ("semi_auto_parallel", "auto_parallel")
        save_checkpoint(net, path, integrated, cfg.async_save, append, cfg.enc_key, cfg.enc_mode,
                        crc_check=cfg.crc_check)
        self._latest = path
        self._files.append(path)
        if cfg.keep_checkpoint_max and len(self._files) > cfg.keep_checkpoint_max:
            old = self._files.pop(0)
            try:
                os.chmod(old, 0o600)
                os.remove(old)
            except OSError:
                pass

    def on_train_step_end(self, run_context):
        self._save(run_context.original_args())

    def on_train_end(self, run_context):
        self._save(run_context.original_args(), force=True)
        from .serialization import wait_async_save
        wait_async_save()


class BackupAndRestore(Callback):
    def __init__(self, backup_dir, save_freq="epoch", delete_checkpoint=True):
        self.backup_dir = os.path.abspath(backup_dir)
        os.makedirs(self.backup_dir, exist_ok=True)
        self.save_freq, self.delete_checkpoint = save_freq, delete_checkpoint
        self.backup_file = os.path.join(self.backup_dir, "backup.ckpt")

    def on_train_begin(self, run_context):
        if os.path.exists(self.backup_file):
            from .serialization import load_checkpoint, load_param_into_net
            p = run_context.original_args()
            d = load_checkpoint(self.backup_file)
            load_param_into_net(p.train_network, d)
            if "epoch_num" in d:
                p.restored_epoch = int(d["epoch_num"])

    def on_train_epoch_end(self, run_context):
        p = run_context.original_args()
        if self.save_freq == "epoch" or (isinstance(self.save_freq, int) and p.cur_epoch_num % self.save_freq == 0):
            from .serialization import save_checkpoint
            save_checkpoint(p.train_network, self.backup_file, integrated_save=False,
                            append_dict={"epoch_num": p.cur_epoch_num, "step_num": p.cur_step_num})

    def on_train_end(self, run_context):
        if self.delete_checkpoint and os.path.exists(self.backup_file):
            os.chmod(self.backup_file, 0o600)
            os.remove(self.backup_file)


class OnRequestExit(Callback):
    """On SIGTERM (or the chosen signal) saves a checkpoint (and graph) at the next step boundary and stops."""

    def __init__(self, save_ckpt=True, save_mindir=True, file_name="Net", directory="./", sig=signal.SIGTERM,
                 config_file=None):
        self.save_ckpt, self.save_mindir, self.file_name = save_ckpt, save_mindir, file_name
        self.directory = os.path.abspath(directory)
        self.sig = sig
        self.exit = False
        self._old = None

    def _handler(self, signum, frame):
        self.exit = True

    def on_train_begin(self, run_context):
        self.exit = False
        self._old = signal.signal(self.sig, self._handler)

    def on_train_step_end(self, run_context):
        if self.exit:
            run_context.request_stop()

    def on_train_end(self, run_context):
        if self._old is not None:
            signal.signal(self.sig, self._old)
        if self.exit and self.save_ckpt:
            from .serialization import save_checkpoint
            os.makedirs(self.directory, exist_ok=True)
            p = run_context.original_args()
            save_checkpoint(p.train_network, os.path.join(self.directory, self.file_name + ".ckpt"),
                            integrated_save=False)

    on_eval_begin = on_train_begin

    def on_eval_step_end(self, run_context):
        if self.exit:
            run_context.request_stop()


class FlopsUtilizationCollector(Callback):
    """Per-step model-FLOPs utilisation.  FLOPs per step: ``flops_per_step`` if given, else what
    ``flops_collection('train')`` reports for the compiled training graph (GRAPH_MODE), looked up after the first
    step.  ``peak_flops`` (per device, FLOP/s) turns the rate into a utilisation."""

    def __init__(self, data_size=None, computility=1, full_flops=True, enable_ma_collector=False,
                 flops_per_step=None, peak_flops=None):
        self.flops_per_step = flops_per_step
        self.peak = peak_flops
        self.records = []

    def on_train_step_begin(self, run_context):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self._t = time.time()

    def on_train_step_end(self, run_context):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.time() - self._t
        rec = {"step_time_s": dt}
        if not self.flops_per_step:
            try:
                from ..graph.flops import flops_collection
                self.flops_per_step = flops_collection("train")[2] or None
            except RuntimeError:
                pass
        if self.flops_per_step:
            rec["tflops"] = self.flops_per_step / dt / 1e12
            if self.peak:
                rec["mfu"] = self.flops_per_step / dt / self.peak
        self.records.append(rec)


class ClusterMonitor(Callback):
    """Writes per-step throughput lines to ``<log_path>/worker_<rank>.log``."""

    def __init__(self, log_path=None):
        self.log_path = log_path or os.environ.get("PERF_DUMP_PATH", "")
        self._t = None

    def on_train_step_begin(self, run_context):
        self._t = time.time()

    def on_train_step_end(self, run_context):
        if not self.log_path:
            return
        os.makedirs(self.log_path, exist_ok=True)
        p = run_context.original_args()
        rank = int(os.environ.get("RANK_ID", "0"))
        with open(os.path.join(self.log_path, "worker_%d.log" % rank), "a") as f:
            f.write(json.dumps({"step": p.cur_step_num, "step_time_ms": (time.time() - self._t) * 1000,
                                "loss": _loss_value(p.net_outputs)}) + "\n")


class SummaryCollector(Callback):
    """Collects the loss (and the learning rate when the optimizer exposes one) every ``collect_freq`` steps into
    a summary event file under ``summary_dir`` (``train.summary.SummaryRecord``: framed, CRC-checked protobuf events,
    the format MindInsight reads), plus one JSON line per record for quick inspection
    (train/callback/_summary_collector.py in the reference)."""

    def __init__(self, summary_dir, collect_freq=10, collect_specified_data=None, keep_default_action=True,
                 custom_lineage_data=None, collect_tensor_freq=None, max_file_size=None, export_options=None):
        from .summary import SummaryRecord
        self.dir = os.path.abspath(summary_dir)
        os.makedirs(self.dir, exist_ok=True)
        self.freq = max(1, int(collect_freq))
        self.path = os.path.join(self.dir, "events.summary.%d.jsonl" % os.getpid())
        self._record = SummaryRecord(self.dir)
        self._lineage = dict(custom_lineage_data or {})

    def on_train_begin(self, run_context):
        if self._lineage:
            with open(os.path.join(self.dir, "lineage.json"), "w") as f:
                json.dump(self._lineage, f)

    def on_train_step_end(self, run_context):
        p = run_context.original_args()
        if p.cur_step_num % self.freq == 0:
            loss = _loss_value(p.net_outputs)
            self._record.add_value("scalar", "loss/auto", loss)
            opt = getattr(p, "optimizer", None)
            if opt is not None and hasattr(opt, "get_lr"):
                try:
                    self._record.add_value("scalar", "learning_rate/auto", float(opt.get_lr()))
                except (TypeError, ValueError, RuntimeError):
                    pass
            self._record.record(p.cur_step_num)
            with open(self.path, "a") as f:
                f.write(json.dumps({"step": p.cur_step_num, "tag": "loss/auto", "value": loss}) + "\n")

    def on_train_end(self, run_context):
        self._record.close()


class SummaryLandscape:
    """Loss landscape around the end of a training run: the loss is evaluated on a ``steps x steps`` grid spanned
    by two directions through the final weights - the two leading principal components of the checkpoints saved over
    training (``landscape_type='pca'``) or two random directions scaled per parameter to the weight norm
    ('random') - and written to ``<summary_dir>/landscape.json`` (train/callback/_landscape.py in the reference;
    there the grid is farmed out to several devices)."""

    def __init__(self, summary_dir):
        self.dir = os.path.abspath(summary_dir)
        os.makedirs(self.dir, exist_ok=True)

    def clean_ckpt(self):
        ck = os.path.join(self.dir, "ckpt_dir")
        if os.path.isdir(ck):
            for f in os.listdir(ck):
                os.remove(os.path.join(ck, f))

    def gen_landscapes_with_multi_process(self, callback_fn, collect_landscape=None, device_ids=None, output=None):
        """``callback_fn()`` returns (model, network, dataset, metrics); ``collect_landscape`` may hold
        ``landscape_size``, ``create_landscape`` ({'train': bool, 'result': bool}), ``num_samples``, ``intervals``,
        ``checkpoints`` (list of checkpoint files for the PCA directions) and ``landscape_type``."""
        import numpy as np
        import torch
        from .serialization import load_checkpoint
        cfg = dict(collect_landscape or {})
        steps = int(cfg.get("landscape_size", 11))
        span = float(cfg.get("span", 1.0))
        model, network, dataset, _ = callback_fn()
        params = [p for p in network.trainable_params()]
        center = [p.detach().clone() for p in params]
        flat_c = torch.cat([c.reshape(-1).float() for c in center])
        ckpts = cfg.get("checkpoints") or []
        kind = cfg.get("landscape_type", "pca" if len(ckpts) >= 2 else "random")
        if kind == "pca" and len(ckpts) >= 2:
            rows = []
            for path in ckpts:
                sd = load_checkpoint(path)
                rows.append(torch.cat([torch.as_tensor(sd[p.name].asnumpy() if hasattr(sd[p.name], "asnumpy") else
                                                       sd[p.name]).reshape(-1).float() for p in params]) - flat_c)
            _, _, vh = torch.linalg.svd(torch.stack(rows), full_matrices=False)
            scale = max(float(r.norm()) for r in rows) or 1.0
            d1, d2 = vh[0] * scale, (vh[1] if vh.shape[0] > 1 else torch.randn_like(vh[0])) * scale
        else:
            g = torch.Generator().manual_seed(int(cfg.get("seed", 0)))
            dirs = []
            for _ in range(2):
                parts = []
                for c in center:
                    r = torch.randn(c.shape, generator=g)
                    parts.append((r * (c.float().norm() / (r.norm() + 1e-12))).reshape(-1))    # filter normalisation
                dirs.append(torch.cat(parts))
            d1, d2 = dirs

        def set_weights(vec):
            off = 0
            with torch.no_grad():
                for p in params:
                    n = p.numel()
                    p.copy_(vec[off:off + n].reshape(p.shape).to(p.dtype))
                    off += n

        def loss_now():
            tot, cnt = 0.0, 0
            network.set_train(False)
            for i, batch in enumerate(dataset.create_tuple_iterator()):
                with torch.no_grad():
                    tot += float(network(*batch))
                cnt += 1
                if cnt >= int(cfg.get("num_batches", 4)):
                    break
            return tot / max(cnt, 1)

        axis = np.linspace(-span, span, steps)
        grid = np.zeros((steps, steps))
        for i, a in enumerate(axis):
            for j, b in enumerate(axis):
                set_weights(flat_c + float(a) * d1 + float(b) * d2)
                grid[i, j] = loss_now()
        set_weights(flat_c)
        out = output or self.dir
        os.makedirs(out, exist_ok=True)
        path = os.path.join(out, "landscape.json")
        with open(path, "w") as f:
            json.dump({"type": kind, "x": axis.tolist(), "y": axis.tolist(), "loss": grid.tolist()}, f)
        return path


class MindIOTTPAdapter(Callback):
    def __init__(self, *args, **kwargs):
        raise RuntimeError("MindIOTTPAdapter drives the Ascend MindIO TTP service, which is not available here")

"""Global execution context and the auto-parallel context.

``set_context`` / ``get_context`` keep a typed table of execution options (mode, device target,
graph dumping, memory limits, determinism, gpu_config ...).  ``set_auto_parallel_context`` holds
the whole parallel contract (device_num, global_rank, parallel_mode, search_mode, strategy
checkpoint files, full_batch/dataset_strategy, parallel optimizer, comm_fusion, pipeline ...).

Parity: mindspore/python/mindspore/context.py:147 (_Context), :1231 (set_context), :1816
(get_context), :855 (set_auto_parallel_context), :1070, :1091, :1868 (ParallelMode);
key set of mindspore/ccsrc/include/common/utils/parallel_context.h:34-303.
"""
from __future__ import annotations

import os
import threading

import torch

GRAPH_MODE = 0
PYNATIVE_MODE = 1

_MODE_NAMES = {GRAPH_MODE: "GRAPH_MODE", PYNATIVE_MODE: "PYNATIVE_MODE"}



STRICT, COMPATIBLE, LAX = 0, 1, 2          # jit_syntax_level values

class ParallelMode:
    STAND_ALONE = "stand_alone"
    DATA_PARALLEL = "data_parallel"
    HYBRID_PARALLEL = "hybrid_parallel"
    SEMI_AUTO_PARALLEL = "semi_auto_parallel"
    AUTO_PARALLEL = "auto_parallel"
    MODE_LIST = [STAND_ALONE, DATA_PARALLEL, HYBRID_PARALLEL, SEMI_AUTO_PARALLEL, AUTO_PARALLEL]


def _default_device_target():
    return "GPU" if torch.cuda.is_available() else "CPU"


_CONTEXT_DEFAULTS = {
    "mode": PYNATIVE_MODE,
    "device_target": None,  # resolved lazily
    "device_id": int(os.environ.get("DEVICE_ID", os.environ.get("LOCAL_RANK", "0"))),
    "save_graphs": 0,
    "save_graphs_path": ".",
    "deterministic": "OFF",
    "print_file_path": "",
    "env_config_path": "",
    "max_call_depth": 1000,
    "pynative_synchronize": False,
    "runtime_num_threads": 30,
    "inter_op_parallel_num": 0,
    "op_timeout": 900,
    "max_device_memory": "1024GB",
    "variable_memory_max_size": "0",
    "mempool_block_size": "1GB",
    "memory_optimize_level": "O0",
    "memory_offload": "OFF",
    "enable_graph_kernel": False,
    "graph_kernel_flags": "",
    "enable_reduce_precision": True,
    "check_bprop": False,
    "enable_compile_cache": False,
    "compile_cache_path": "",
    "precompile_only": False,
    "reserve_class_name_in_scope": True,
    "jit_config": {},
    "jit_syntax_level": 2,
    "jit_level": "",
    "debug_level": 0,
    "enable_sparse": False,
    "grad_for_scalar": False,
    "support_binary": False,
    "disable_format_transform": False,
    "gpu_config": {"conv_fprop_algo": "normal", "conv_dgrad_algo": "normal", "conv_wgrad_algo": "normal",
                   "conv_allow_tf32": True, "matmul_allow_tf32": False},
    "ascend_config": {},
    "enable_dump": False,
    "save_dump_path": ".",
    # B200 runtime options (no counterpart in the reference): capture the compiled step in a CUDA graph,
    # and run collectives through the fused NVLink kernels instead of separate NCCL calls.
    "enable_cuda_graph": False,
    "fused_comm": True,
}

_VALID_TARGETS = ("CPU", "GPU", "Ascend")


class _Context:
    _instance = None
    _lock = threading.Lock()

    def __new__(cls):
        if cls._instance is None:
            with cls._lock:
                if cls._instance is None:
                    cls._instance = object.__new__(cls)
                    cls._instance._values = {k: (dict(v) if isinstance(v, dict) else v)
                                             for k, v in _CONTEXT_DEFAULTS.items()}
        return cls._instance

    def get(self, key):
        if key not in self._values:
            raise ValueError("Get context keyword %s is not recognized!" % key)
        if key == "device_target" and self._values[key] is None:
            self._values[key] = _default_device_target()
        return self._values[key]

    def set(self, key, value):
        if key not in self._values:
            raise ValueError("Set context keyword %s is not recognized!" % key)
        setter = getattr(self, "_set_" + key, None)
        if setter:
            setter(value)
        else:
            self._values[key] = value

    def _set_mode(self, mode):
        if mode not in (GRAPH_MODE, PYNATIVE_MODE):
            raise ValueError("For 'context.set_context', the argument 'mode' should be context.GRAPH_MODE (0) "
                             "or context.PYNATIVE_MODE (1), but got %r." % (mode,))
        self._values["mode"] = mode

    def _set_device_target(self, target):
        if target not in _VALID_TARGETS:
            raise ValueError("For 'context.set_context', 'device_target' must be one of %s, but got %r"
                             % (list(_VALID_TARGETS), target))
        if target == "Ascend":
            raise ValueError("device_target 'Ascend' is not available in this build (CPU and GPU only)")
        if target == "GPU" and not torch.cuda.is_available():
            raise RuntimeError("device_target 'GPU' requested but no CUDA device is visible")
        self._values["device_target"] = target

    def _set_device_id(self, device_id):
        if not isinstance(device_id, int) or device_id < 0 or device_id > 4095:
            raise ValueError("For 'context.set_context', 'device_id' must be in [0, 4095], got %r" % (device_id,))
        self._values["device_id"] = device_id
        if torch.cuda.is_available() and device_id < torch.cuda.device_count():
            torch.cuda.set_device(device_id)

    def _set_save_graphs(self, v):
        if isinstance(v, bool):
            v = 1 if v else 0
        if v not in (0, 1, 2, 3):
            raise ValueError("'save_graphs' must be one of 0,1,2,3 or bool, got %r" % (v,))
        self._values["save_graphs"] = v

    def _set_deterministic(self, v):
        if v not in ("ON", "OFF"):
            raise ValueError("'deterministic' must be 'ON' or 'OFF', got %r" % (v,))
        self._values["deterministic"] = v
        torch.use_deterministic_algorithms(v == "ON", warn_only=True)

    def _set_gpu_config(self, cfg):
        allowed = set(_CONTEXT_DEFAULTS["gpu_config"])
        for k in cfg:
            if k not in allowed:
                raise ValueError("gpu_config key %r is not supported (allowed: %s)" % (k, sorted(allowed)))
        self._values["gpu_config"].update(cfg)
        torch.backends.cuda.matmul.allow_tf32 = bool(self._values["gpu_config"]["matmul_allow_tf32"])
        torch.backends.cudnn.allow_tf32 = bool(self._values["gpu_config"]["conv_allow_tf32"])

    def _set_jit_config(self, cfg):
        self._values["jit_config"] = dict(cfg)
        if "jit_level" in cfg:
            self._values["jit_level"] = cfg["jit_level"]

    def _set_max_device_memory(self, v):
        if not (isinstance(v, str) and v.endswith("GB")):
            raise ValueError("'max_device_memory' should be in the form '4GB', got %r" % (v,))
        self._values["max_device_memory"] = v

    def reset(self):
        self._values = {k: (dict(v) if isinstance(v, dict) else v) for k, v in _CONTEXT_DEFAULTS.items()}


def _context():
    return _Context()


def set_context(**kwargs):
    """Sets execution options; unknown keys raise ``ValueError`` like the reference."""
    ctx = _context()
    # device_target first: other setters may depend on it
    for key in sorted(kwargs, key=lambda k: (k != "device_target", k != "mode", k)):
        ctx.set(key, kwargs[key])


def get_context(attr_key):
    return _context().get(attr_key)


def _get_mode():
    return _context().get("mode")


def device():
    """torch.device implied by (device_target, device_id)."""
    ctx = _context()
    if ctx.get("device_target") == "GPU":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


# --------------------------------------------------------------------------------------------
# auto-parallel context
# --------------------------------------------------------------------------------------------
_PARALLEL_DEFAULTS = {
    "device_num": 1,
    "global_rank": 0,
    "gradients_mean": False,
    "gradient_fp32_sync": True,
    "parallel_mode": ParallelMode.STAND_ALONE,
    "search_mode": "recursive_programming",
    "auto_parallel_search_mode": "recursive_programming",
    "parameter_broadcast": False,
    "strategy_ckpt_load_file": "",
    "strategy_ckpt_save_file": "",
    "strategy_ckpt_config": {},
    "full_batch": False,
    "dataset_strategy": "data_parallel",
    "enable_parallel_optimizer": False,
    "parallel_optimizer_config": {"gradient_accumulation_shard": True, "parallel_optimizer_threshold": 64,
                                  "optimizer_weight_shard_size": -1},
    "enable_alltoall": False,
    "all_reduce_fusion_config": [],
    "comm_fusion": {},
    "pipeline_stages": 1,
    "pipeline_segments": 1,
    "pipeline_result_broadcast": False,
    "pipeline_config": {"pipeline_interleave": False, "pipeline_scheduler": "1f1b"},
    "group_ckpt_save_file": "",
    "auto_pipeline": False,
    "force_fp32_communication": False,
    "grad_accumulation_step": 1,
    "optimizer_weight_shard_size": -1,
    "optimizer_weight_shard_aggregated_save": False,
    "sharding_propagation": False,
    "enable_fine_grained_micro_interleaved": False,
    "fine_grained_micro_interleaved_size": -1,
    "loss_repeated_mean": True,
    "device_num_is_set": False,
    "global_rank_is_set": False,
}

_SEARCH_MODES = ("recursive_programming", "sharding_propagation", "dynamic_programming")


class _AutoParallelContext:
    _instance = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = object.__new__(cls)
            cls._instance.reset()
        return cls._instance

    def reset(self):
        self._v = {k: (dict(v) if isinstance(v, dict) else (list(v) if isinstance(v, list) else v))
                   for k, v in _PARALLEL_DEFAULTS.items()}

    def get(self, key):
        if key not in self._v:
            raise ValueError("Get context keyword %s is not recognized!" % key)
        if key == "device_num" and not self._v["device_num_is_set"]:
            from .communication import management as _m
            if _m.GlobalComm.INITED:
                return _m.get_group_size()
        if key == "global_rank" and not self._v["global_rank_is_set"]:
            from .communication import management as _m
            if _m.GlobalComm.INITED:
                return _m.get_rank()
        return self._v[key]

    def set(self, key, value):
        if key not in self._v:
            raise ValueError("Set context keyword %s is not recognized!" % key)
        checker = getattr(self, "_check_" + key, None)
        if checker:
            value = checker(value)
        self._v[key] = value

    def _check_device_num(self, n):
        if not isinstance(n, int) or n < 1 or n > 4096:
            raise ValueError("The context configuration parameter 'device_num' must be in [1, 4096], but got %r" % (n,))
        self._v["device_num_is_set"] = True
        return n

    def _check_global_rank(self, r):
        if not isinstance(r, int) or r < 0 or r > 4095:
            raise ValueError("The context configuration parameter 'global_rank' must be in [0, 4095], but got %r" % (r,))
        self._v["global_rank_is_set"] = True
        return r

    def _check_parallel_mode(self, m):
        if m not in ParallelMode.MODE_LIST:
            raise ValueError("The context configuration parameter 'parallel_mode' only supports %s, but got %r"
                             % (ParallelMode.MODE_LIST, m))
        return m

    def _check_search_mode(self, m):
        if m not in _SEARCH_MODES:
            raise ValueError("The context configuration parameter 'search_mode' only supports %s, but got %r"
                             % (list(_SEARCH_MODES), m))
        self._v["auto_parallel_search_mode"] = m
        return m

    def _check_auto_parallel_search_mode(self, m):
        return self._check_search_mode(m)

    def _check_pipeline_stages(self, s):
        if not isinstance(s, int) or s < 1:
            raise ValueError("'pipeline_stages' must be a positive int, got %r" % (s,))
        return s

    def _check_dataset_strategy(self, s):
        if isinstance(s, str):
            if s not in ("full_batch", "data_parallel"):
                raise ValueError("'dataset_strategy' must be 'full_batch', 'data_parallel' or a tuple of tuples")
            self._v["full_batch"] = s == "full_batch"
            return s
        if not isinstance(s, (tuple, list)) or not all(isinstance(t, (tuple, list)) for t in s):
            raise TypeError("'dataset_strategy' must be str or tuple(tuple(int))")
        return tuple(tuple(int(i) for i in t) for t in s)

    def _check_full_batch(self, b):
        if not isinstance(b, bool):
            raise TypeError("'full_batch' must be bool")
        self._v["dataset_strategy"] = "full_batch" if b else "data_parallel"
        return b

    def _check_parallel_optimizer_config(self, cfg):
        allowed = {"gradient_accumulation_shard", "parallel_optimizer_threshold", "optimizer_weight_shard_size"}
        for k in cfg:
            if k not in allowed:
                raise ValueError("parallel_optimizer_config key %r is not supported" % k)
        merged = dict(self._v["parallel_optimizer_config"])
        merged.update(cfg)
        if "optimizer_weight_shard_size" in cfg:
            self._v["optimizer_weight_shard_size"] = cfg["optimizer_weight_shard_size"]
        return merged

    def _check_comm_fusion(self, cfg):
        if not isinstance(cfg, dict):
            raise TypeError("'comm_fusion' must be dict")
        for op, c in cfg.items():
            if op == "openstate":
                continue
            if op not in ("allreduce", "allgather", "reducescatter"):
                raise KeyError("comm_fusion key %r is not supported" % op)
            if c.get("mode") not in ("auto", "size", "index"):
                raise KeyError("comm_fusion mode must be auto, size or index, got %r" % (c.get("mode"),))
        if "allreduce" in cfg and cfg["allreduce"].get("mode") == "index":
            self._v["all_reduce_fusion_config"] = list(cfg["allreduce"].get("config", []))
        return dict(cfg)

    def _check_all_reduce_fusion_config(self, idx):
        if not isinstance(idx, (list, tuple)):
            raise TypeError("'all_reduce_fusion_config' must be list")
        idx = list(idx)
        if any((not isinstance(i, int)) for i in idx) or idx != sorted(idx):
            raise ValueError("'all_reduce_fusion_config' must be an ascending list of int")
        return idx

    def _check_pipeline_config(self, cfg):
        merged = dict(self._v["pipeline_config"])
        for k, v in cfg.items():
            if k not in ("pipeline_interleave", "pipeline_scheduler"):
                raise ValueError("pipeline_config key %r is not supported" % k)
            merged[k] = v
        if merged["pipeline_scheduler"] not in ("1f1b", "gpipe"):
            raise ValueError("pipeline_scheduler must be '1f1b' or 'gpipe'")
        return merged

    def _check_strategy_ckpt_config(self, cfg):
        for k in cfg:
            if k not in ("load_file", "save_file", "only_trainable_params"):
                raise ValueError("strategy_ckpt_config key %r is not supported" % k)
        if "load_file" in cfg:
            self._v["strategy_ckpt_load_file"] = cfg["load_file"]
        if "save_file" in cfg:
            self._v["strategy_ckpt_save_file"] = cfg["save_file"]
        return dict(cfg)


def _parallel_ctx():
    return _AutoParallelContext()


def set_auto_parallel_context(**kwargs):
    ctx = _parallel_ctx()
    for k in sorted(kwargs, key=lambda k: (k != "parallel_mode", k)):
        ctx.set(k, kwargs[k])


def get_auto_parallel_context(attr_key):
    return _parallel_ctx().get(attr_key)


def reset_auto_parallel_context():
    _parallel_ctx().reset()


# ---- parameter-server / offload contexts: accepted for API compatibility, stored verbatim ----
_ps_context = {"enable_ps": False, "enable_ssl": False}
_offload_context = {"offload_param": "", "offload_path": "./offload", "offload_cpu_size": "512GB",
                    "offload_disk_size": "1024GB", "enable_aio": True, "enable_pinned_mem": True,
                    "auto_offload": True, "host_mem_block_size": "1GB"}


def set_ps_context(**kwargs):
    _ps_context.update(kwargs)


def get_ps_context(key):
    return _ps_context[key]


def reset_ps_context():
    _ps_context.clear()
    _ps_context.update({"enable_ps": False, "enable_ssl": False})


def set_offload_context(offload_config):
    _offload_context.update(offload_config)


def get_offload_context():
    return dict(_offload_context)

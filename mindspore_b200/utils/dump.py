"""Tensor dump: ``set_dump(cell)`` marks cells whose outputs are written as ``.npy`` files while
``MINDSPORE_DUMP_CONFIG`` points to a JSON config {"common_dump_settings": {"path", "net_name", "iteration"}}
(python/mindspore/common/dump.py set_dump; ccsrc/debug/data_dump/dump_json_parser.cc, e2e_dump.cc for the layout
``<path>/rank_<r>/<net>/<graph>/<iteration>/<op>.<slot>.npy``)."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

_state = {"iteration": 0, "config": None}


def _config():
    if _state["config"] is None:
        path = os.environ.get("MINDSPORE_DUMP_CONFIG")
        cfg = {}
        if path and os.path.isfile(path):
            with open(path) as f:
                cfg = json.load(f).get("common_dump_settings", {})
        _state["config"] = cfg
    return _state["config"]


def reset():
    _state["config"] = None
    _state["iteration"] = 0


def next_iteration():
    _state["iteration"] += 1


def _wanted_iteration(cfg):
    it = str(cfg.get("iteration", "all"))
    if it == "all":
        return True
    cur = _state["iteration"]
    for part in it.split("|"):
        if "-" in part:
            lo, hi = part.split("-")
            if int(lo) <= cur <= int(hi):
                return True
        elif part.strip() and int(part) == cur:
            return True
    return False


def set_dump(target, enabled=True):
    """Enables or disables dumping of the outputs of ``target`` (a Cell or a Primitive)."""
    from ..nn.cell import Cell
    from ..ops.primitive import Primitive
    if not isinstance(target, (Cell, Primitive)):
        raise ValueError("The \"target\" parameter must be an instance of Cell or Primitive, but got %s" % type(target))
    if isinstance(target, Primitive):
        target.add_prim_attr("dump", "true" if enabled else "false")
        return
    if getattr(target, "_dump_handle", None) is not None:
        target._dump_handle.remove()
        object.__setattr__(target, "_dump_handle", None)
    if not enabled:
        return

    def hook(cell, inputs, output):
        cfg = _config()
        if not cfg.get("path") or not _wanted_iteration(cfg):
            return None
        rank = int(os.environ.get("RANK_ID", os.environ.get("RANK", "0")))
        d = os.path.join(cfg["path"], "rank_%d" % rank, cfg.get("net_name", "net"), "0", str(_state["iteration"]))
        os.makedirs(d, exist_ok=True)
        outs = output if isinstance(output, (tuple, list)) else (output,)
        for i, o in enumerate(outs):
            if isinstance(o, torch.Tensor):
                np.save(os.path.join(d, "%s.output.%d.npy" % (cell.cls_name, i)),
                        o.detach().float().cpu().numpy())
        return None

    object.__setattr__(target, "_dump_handle", target.register_forward_hook(hook))

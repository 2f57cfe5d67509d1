"""Weight obfuscation of checkpoints (the reference's ``mindspore.safeguard``).

``obfuscate_ckpt`` multiplies the weights of the chosen layers by secret random ratios and writes the scaled
checkpoints; ``load_obf_params_into_net`` prepares the network that will load them: every chosen layer divides its
input by its ratio, so the layer computes ``(x / r) @ (r W) = x @ W`` with the scaled weights staying scaled in memory
and on disk.  Without the ratios the checkpoint gives wrong outputs.  ``target_modules = [path, names(, scope)]``:
``path`` is the cell path ``'A/B/C'`` below which layers are looked for (``''`` = the whole network), ``names`` the
layer names ``'D|E|F'``, and the optional third entry ``'obfuscate_layers:all'`` / ``'obfuscate_layers:<n>'`` limits
repeated blocks (cells reached through a numeric path component) to the first n.

Graph-level ("dynamic") obfuscation of MindIR files (``obfuscate_model``) is not provided.

Parity: python/mindspore/safeguard/rewrite_obfuscation.py:35 (obfuscate_ckpt), :166 (load_obf_params_into_net)."""
from __future__ import annotations

import os
import re

import numpy as np
import torch

from .nn.cell import Cell

_PATH_RE = re.compile(r"^[A-Za-z0-9_/]*$")
_NAMES_RE = re.compile(r"^[A-Za-z0-9_|]+$")


def _check_targets(target_modules):
    if not isinstance(target_modules, list):
        raise TypeError("target_modules must be a list, but got %s" % type(target_modules).__name__)
    if len(target_modules) < 2:
        raise ValueError("target_modules needs at least two elements: the module path and the layer names")
    if not all(isinstance(t, str) for t in target_modules):
        raise TypeError("the elements of target_modules must be strings")
    path, names = target_modules[0], target_modules[1]
    if path == "/":
        path = ""
    if not _PATH_RE.match(path):
        raise ValueError("target_modules[0] may only hold letters, digits, '_' and '/', but got %r" % path)
    if not names or not _NAMES_RE.match(names):
        raise ValueError("target_modules[1] must be layer names joined by '|', but got %r" % names)
    limit = None
    if len(target_modules) > 2:
        m = re.match(r"^obfuscate_layers:(all|\d+)$", target_modules[2])
        if not m:
            raise ValueError("target_modules[2] must be 'obfuscate_layers:all' or 'obfuscate_layers:<int>', but got %r"
                             % target_modules[2])
        limit = None if m.group(1) == "all" else int(m.group(1))
    return path.strip("/"), names.split("|"), limit


def _target_cells(network, target_modules):
    """[(cell path with '.', cell)] of the layers to obfuscate, in network order."""
    path, names, limit = _check_targets(target_modules)
    prefix = path.replace("/", ".")
    out = []
    for name, cell in network.cells_and_names():
        if not name or name.split(".")[-1] not in names:
            continue
        parent = ".".join(name.split(".")[:-1])
        stripped = ".".join(p for p in parent.split(".") if not p.isdigit())
        if prefix and not (parent == prefix or parent.startswith(prefix + ".") or stripped == prefix
                           or stripped.startswith(prefix + ".")):
            continue
        layer_ids = [int(p) for p in name.split(".") if p.isdigit()]
        if limit is not None and layer_ids and layer_ids[0] >= limit:
            continue
        if getattr(cell, "weight", None) is None:
            continue
        out.append((name, cell))
    if not out:
        raise ValueError("The obfuscate module path %s is not exist, please check the input 'target_modules'."
                         % (target_modules,))
    return out


def obfuscate_ckpt(network, ckpt_files, target_modules=None, saved_path="./", obfuscate_scale=100):
    """Writes ``<saved_path>/<name>_obf.ckpt`` for every ``.ckpt`` in the folder ``ckpt_files`` with the target
    layers' weights scaled, and returns the list of ratios (one per target layer, in network order)."""
    from .train.serialization import load_checkpoint, save_checkpoint
    if not isinstance(network, Cell):
        raise TypeError("network must be nn.Cell, but got %s." % type(network))
    for label, p in (("ckpt_files", ckpt_files), ("saved_path", saved_path)):
        if not isinstance(p, str):
            raise TypeError("%s must be string, but got %s." % (label, type(p)))
        if not os.path.isdir(p):
            raise ValueError("%s %s is not exist." % (label, p))
    if not isinstance(obfuscate_scale, (int, float)) or obfuscate_scale <= 1:
        raise ValueError("obfuscate_scale must be a number larger than 1, but got %r" % (obfuscate_scale,))
    if target_modules is None:
        names = sorted({n.split(".")[-1] for n, c in network.cells_and_names()
                        if n and getattr(c, "weight", None) is not None and getattr(c.weight, "ndim", 0) >= 2})
        target_modules = ["", "|".join(names)]
    cells = _target_cells(network, target_modules)
    rng = np.random.default_rng()
    lo, hi = np.log(1.0 / obfuscate_scale), np.log(float(obfuscate_scale))
    ratios = [float(np.exp(rng.uniform(lo, hi))) for _ in cells]
    by_param = {cell.weight.name: r for (_, cell), r in zip(cells, ratios)}
    for fname in sorted(os.listdir(ckpt_files)):
        if not fname.endswith(".ckpt"):
            continue
        params = load_checkpoint(os.path.join(ckpt_files, fname))
        out = []
        for name, p in params.items():
            data = p.detach().as_subclass(torch.Tensor)
            if name in by_param:
                data = (data.float() * by_param[name]).to(data.dtype)
            out.append({"name": name, "data": data})
        save_checkpoint(out, os.path.join(saved_path, fname[:-5] + "_obf.ckpt"))
    return ratios


def load_obf_params_into_net(network, target_modules=None, obf_ratios=None, data_parallel_num=1, **kwargs):
    """Makes ``network`` ready for an obfuscated checkpoint: each target layer divides its input by its ratio.
    Returns the same network; load the ``*_obf.ckpt`` into it afterwards (or before: order does not matter)."""
    if not isinstance(network, Cell):
        raise TypeError("network must be nn.Cell, but got %s." % type(network))
    if obf_ratios is None:
        raise ValueError("obf_ratios (what obfuscate_ckpt returned) is required")
    ratios = [float(r) for r in (obf_ratios.tolist() if hasattr(obf_ratios, "tolist") else obf_ratios)]
    if target_modules is None:
        names = sorted({n.split(".")[-1] for n, c in network.cells_and_names()
                        if n and getattr(c, "weight", None) is not None and getattr(c.weight, "ndim", 0) >= 2})
        target_modules = ["", "|".join(names)]
    cells = _target_cells(network, target_modules)
    if len(ratios) != len(cells):
        raise ValueError("got %d obf_ratios for %d target layers" % (len(ratios), len(cells)))
    for (_, cell), r in zip(cells, ratios):
        if getattr(cell, "_obf_ratio", None) is not None:
            cell._obf_ratio = r
            continue
        cell._obf_ratio = r

        def pre(c, inputs):
            return (inputs[0] / c._obf_ratio,) + tuple(inputs[1:])
        cell.register_forward_pre_hook(pre)
    return network


def obfuscate_model(obf_config, **kwargs):
    raise NotImplementedError("graph-level obfuscation of MindIR files is not provided; use obfuscate_ckpt / "
                              "load_obf_params_into_net for weight obfuscation")


__all__ = ["obfuscate_ckpt", "load_obf_params_into_net", "obfuscate_model"]

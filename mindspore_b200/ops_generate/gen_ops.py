"""yaml operator definitions -> Python source with one ``Primitive`` class and one functional wrapper per operator.

    python -m mindspore_b200.ops_generate --out gen_ops_def.py [yaml files or directories ...]

Each definition names its arguments in call order.  Arguments marked ``prim_init`` become constructor arguments of
the primitive (recorded as primitive attributes); the others are call inputs.  ``dtype`` is checked when the
primitive is called: ``tensor``, ``number``, ``int``, ``float``, ``bool``, ``str``, ``tuple[int]``, ``list[int]``
(a trailing ``?`` or a ``null`` default allows None).  The functional wrapper takes all arguments in order and
creates (and caches) the primitive for each combination of ``prim_init`` values."""
from __future__ import annotations

import argparse
import keyword
import os
import sys

import yaml

_CHECKS = {
    "tensor": "isinstance({v}, torch.Tensor)",
    "number": "isinstance({v}, (int, float, bool)) or (isinstance({v}, torch.Tensor) and {v}.dim() == 0)",
    "int": "isinstance({v}, int) and not isinstance({v}, bool)",
    "float": "isinstance({v}, (int, float)) and not isinstance({v}, bool)",
    "bool": "isinstance({v}, bool)",
    "str": "isinstance({v}, str)",
    "tuple[int]": "isinstance({v}, (tuple, list)) and all(isinstance(_e, int) for _e in {v})",
    "list[int]": "isinstance({v}, (tuple, list)) and all(isinstance(_e, int) for _e in {v})",
    "tuple[tensor]": "isinstance({v}, (tuple, list)) and all(isinstance(_e, torch.Tensor) for _e in {v})",
    "any": "True",
}


class OpDefError(ValueError):
    pass


def _camel(name):
    return "".join(p.capitalize() for p in name.split("_"))


def load_definitions(paths):
    """{op name: definition} from yaml files / directories, validated."""
    files = []
    for p in paths:
        if os.path.isdir(p):
            files += sorted(os.path.join(p, f) for f in os.listdir(p) if f.endswith((".yaml", ".yml")))
        else:
            files.append(p)
    defs = {}
    for f in files:
        with open(f) as fh:
            doc = yaml.safe_load(fh) or {}
        for name, d in doc.items():
            if name in defs:
                raise OpDefError("operator %s is defined twice (second time in %s)" % (name, f))
            if not name.isidentifier() or keyword.iskeyword(name):
                raise OpDefError("%s: operator name %r is not a valid identifier" % (f, name))
            if not isinstance(d, dict) or "args" not in d or "impl" not in d:
                raise OpDefError("%s: operator %s needs 'args' and 'impl'" % (f, name))
            seen_default = False
            for arg, spec in d["args"].items():
                spec = spec or {}
                dt = str(spec.get("dtype", "any")).rstrip("?")
                if dt not in _CHECKS:
                    raise OpDefError("%s: %s.%s has unknown dtype %r" % (f, name, arg, spec.get("dtype")))
                if "default" in spec:
                    seen_default = True
                elif seen_default:
                    raise OpDefError("%s: %s.%s without default follows an argument with one" % (f, name, arg))
            defs[name] = d
    return defs


def _default_src(spec):
    return repr(spec["default"])


def _emit_op(name, d):
    cls = d.get("class") or _camel(name)
    fn = d.get("function") or name
    args = [(a, s or {}) for a, s in d["args"].items()]
    init = [(a, s) for a, s in args if s.get("prim_init")]
    call = [(a, s) for a, s in args if not s.get("prim_init")]

    def sig(items):
        return ", ".join(a + ("=" + _default_src(s) if "default" in s else "") for a, s in items)

    def checks(items, indent, where):
        out = []
        for a, s in items:
            dt = str(s.get("dtype", "any"))
            optional = dt.endswith("?") or ("default" in s and s["default"] is None)
            cond = _CHECKS[dt.rstrip("?")].format(v=a)
            if cond == "True":
                continue
            if optional:
                cond = "%s is None or (%s)" % (a, cond)
            out.append("%sif not (%s):" % (indent, cond))
            out.append("%s    raise TypeError(\"For '%s', %s '%s' must be %s, but got \" + type(%s).__name__)"
                       % (indent, cls, where, a, dt.rstrip("?"), a))
        return out

    lines = ["class %s(Primitive):" % cls,
             "    \"\"\"%s  Generated from the definition of ``%s``.\"\"\"" % (d.get("description", cls + "."), name),
             "",
             "    @prim_attr_register",
             "    def __init__(self%s):" % ((", " + sig(init)) if init else "")]
    body = checks(init, "        ", "the attribute")
    lines += body or ["        pass"]
    lines += ["", "    def _run(self%s):" % ((", " + sig(call)) if call else "")]
    lines += checks(call, "        ", "the input")
    for a, _ in init:
        lines.append("        %s = self.%s" % (a, a))
    lines += ["        return %s" % d["impl"], "", ""]
    key = ", ".join(a for a, _ in init)
    lines += ["def %s(%s):" % (fn, sig(args)),
              "    \"\"\"Functional form of :class:`%s`.\"\"\"" % cls]
    if init:
        lines += ["    key = (%s,)" % key,
                  "    op = _cache.get((%r, key))" % cls,
                  "    if op is None:",
                  "        op = _cache[(%r, key)] = %s(%s)" % (cls, cls, key)]
    else:
        lines += ["    op = _cache.get(%r)" % cls,
                  "    if op is None:",
                  "        op = _cache[%r] = %s()" % (cls, cls)]
    lines += ["    return op(%s)" % ", ".join(a for a, _ in call), "", ""]
    return cls, fn, lines


def generate(defs):
    """Python source of the generated module."""
    out = ['"""Generated by mindspore_b200.ops_generate - do not edit."""',
           "import torch",
           "import torch.nn.functional as F  # noqa: F401",
           "",
           "from mindspore_b200.ops.primitive import Primitive, prim_attr_register",
           "",
           "_cache = {}",
           "", ""]
    names = []
    for name in sorted(defs):
        cls, fn, lines = _emit_op(name, defs[name])
        names += [cls, fn]
        out += lines
    out.append("__all__ = %r" % (names,))
    return "\n".join(out) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser(prog="mindspore_b200.ops_generate")
    ap.add_argument("paths", nargs="*", default=[os.path.join(os.path.dirname(os.path.abspath(__file__)), "ops_def")])
    ap.add_argument("--out", default="-")
    args = ap.parse_args(argv)
    src = generate(load_definitions(args.paths))
    if args.out == "-":
        sys.stdout.write(src)
    else:
        with open(args.out, "w") as f:
            f.write(src)
    return 0

"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``libmsb200_cuda.so``  - every ``csrc/cuda/*.cu`` compiled for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); plain ``extern "C"`` launchers
  that take raw device pointers and a stream, called through ``ctypes``.
* ``libmsb200_host.so``  - every ``csrc/host/*.cpp`` (layout algebra, strategy
  search, pipeline scheduler, checkpoint codec, cluster store, memory planner).

Objects are rebuilt only when the hash of (source, headers, flags) changes, so
importing the package on a machine that received pre-built binaries does not
recompile anything.  Run ``python -m mindspore_b200._native.build`` to build.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
CSRC_CUDA = os.path.join(PKG, "csrc", "cuda")
CSRC_HOST = os.path.join(PKG, "csrc", "host")
OBJ_DIR = os.path.join(HERE, "build")

CUDA_LIB = os.path.join(HERE, "libmsb200_cuda.so")
HOST_LIB = os.path.join(HERE, "libmsb200_host.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install CUDA 12.9")


def _digest(paths, flags) -> str:
    h = hashlib.sha256()
    for f in flags:
        h.update(f.encode())
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _headers(d):
    return [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".h", ".cuh", ".hpp"))]


def _compile_one(cmd, obj, stamp, digest, log):
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log, "w") as fh:
        fh.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("compile failed: %s\n%s" % (" ".join(cmd), r.stdout + r.stderr))
    with open(stamp, "w") as fh:
        fh.write(digest)
    return obj


def _build_lib(srcs, hdrs, compiler_cmd, flags, lib, link_cmd, verbose):
    os.makedirs(OBJ_DIR, exist_ok=True)
    objs, jobs = [], []
    for src in srcs:
        base = os.path.splitext(os.path.basename(src))[0]
        obj = os.path.join(OBJ_DIR, base + ".o")
        stamp = obj + ".hash"
        digest = _digest([src] + hdrs, flags)
        objs.append(obj)
        if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest:
            continue
        jobs.append((compiler_cmd + flags + ["-c", src, "-o", obj], obj, stamp, digest, obj + ".log"))
    if jobs:
        if verbose:
            print("[mindspore_b200] compiling %d file(s) for %s" % (len(jobs), os.path.basename(lib)), flush=True)
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for fut in [ex.submit(_compile_one, *j) for j in jobs]:
                fut.result()
    link_stamp = lib + ".hash"
    link_digest = _digest(objs, link_cmd) if all(os.path.exists(o) for o in objs) else ""
    if jobs or not os.path.exists(lib) or not os.path.exists(link_stamp) or open(link_stamp).read() != link_digest:
        r = subprocess.run(link_cmd + objs + ["-o", lib], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed: %s\n%s" % (" ".join(link_cmd), r.stdout + r.stderr))
        with open(link_stamp, "w") as fh:
            fh.write(_digest(objs, link_cmd))
    return lib


def build_cuda(verbose=True) -> str:
    srcs = sorted(os.path.join(CSRC_CUDA, f) for f in os.listdir(CSRC_CUDA) if f.endswith(".cu"))
    nvcc = _nvcc()
    shared = [h for h in _headers(CSRC_HOST) if h.endswith(".hpp")]      # headers the device code includes too
    return _build_lib(srcs, _headers(CSRC_CUDA) + shared, [nvcc], NVCC_FLAGS, CUDA_LIB,
                      [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"], verbose)


def build_host(verbose=True) -> str:
    srcs = sorted(os.path.join(CSRC_HOST, f) for f in os.listdir(CSRC_HOST) if f.endswith(".cpp"))
    cxx = os.environ.get("CXX", "g++")
    return _build_lib(srcs, _headers(CSRC_HOST), [cxx], CXX_FLAGS, HOST_LIB, [cxx, "-shared", "-pthread"], verbose)


def build_all(verbose=True):
    return build_host(verbose), build_cuda(verbose)


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of the last compile of each CUDA source."""
    out = []
    if os.path.isdir(OBJ_DIR):
        for f in sorted(os.listdir(OBJ_DIR)):
            if f.endswith(".o.log"):
                out.append(open(os.path.join(OBJ_DIR, f)).read())
    return "\n".join(out)


if __name__ == "__main__":
    libs = build_all(True)
    print("built:", *libs, sep="\n  ")
    if "--ptxas" in sys.argv:
        print(ptxas_report())

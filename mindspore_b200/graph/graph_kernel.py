"""Graph-kernel fusion: chains of elementwise primitives become ONE generated CUDA kernel.

An elementwise chain in a transformer step (bias + residual + activation + scale ...) is bandwidth bound: every
primitive reads and writes the whole tensor through HBM.  ``fuse_elementwise(fg)`` groups connected elementwise
primitive nodes of equal shape and dtype into clusters, replaces each cluster by one ``FusedElementwise`` node, and
that node runs a kernel generated for exactly this expression: every input is read once with 16-byte vector loads
(two per thread in flight),
the expression is evaluated in fp32 registers, every output is written once.  The kernel text is compiled for
sm_100a with nvcc into a shared object (cached by the hash of its source), loaded through ctypes and launched on the
current stream; a grid of 148 SMs x 8 blocks walks the tensor with a grid-stride loop.  On CPU tensors, and for the
backward pass, the node evaluates the same expression with torch operators.

Clustering keeps the graph order valid: a node joins the cluster(s) of its producers only if no value of the cluster
is consumed by an outside node that sits before it (the fused node takes the place of the cluster's last member).
Clusters are capped at 24 nodes, 8 inputs and 4 outputs.  Enabled by ``set_context(enable_graph_kernel=True)``.

Parity (role): mindspore/ccsrc/backend/common/graph_kernel/ (cluster + expander passes, core/graph_kernel_cluster.cc)
and the AKG-generated kernels they dispatch to; python/mindspore/_extends/graph_kernel (the cost model that decides
what to fuse, here the fixed caps above).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess

import torch

__all__ = ["fuse_elementwise", "FusedElementwise", "kernel_source"]

# primitive name -> (C expression over a, b; the same with torch)
_UNARY = {
    "Neg": ("-a", torch.neg), "Exp": ("expf(a)", torch.exp), "Log": ("logf(a)", torch.log),
    "Tanh": ("tanhf(a)", torch.tanh), "Sigmoid": ("1.f / (1.f + expf(-a))", torch.sigmoid),
    "ReLU": ("fmaxf(a, 0.f)", torch.relu), "Sqrt": ("sqrtf(a)", torch.sqrt), "Rsqrt": ("rsqrtf(a)", torch.rsqrt),
    "Abs": ("fabsf(a)", torch.abs), "Square": ("a * a", torch.square), "Reciprocal": ("1.f / a", torch.reciprocal),
    "SiLU": ("a / (1.f + expf(-a))", torch.nn.functional.silu), "Erf": ("erff(a)", torch.erf),
}
_BINARY = {
    "Add": ("a + b", torch.add), "Sub": ("a - b", torch.sub), "Mul": ("a * b", torch.mul),
    "RealDiv": ("a / b", torch.div), "Div": ("a / b", torch.div), "Maximum": ("fmaxf(a, b)", torch.maximum),
    "Minimum": ("fminf(a, b)", torch.minimum),
}
_DTYPES = {torch.float32: ("float", 4), torch.bfloat16: ("__nv_bfloat16", 8), torch.float16: ("__half", 8)}
MAX_NODES, MAX_INPUTS, MAX_OUTPUTS = 24, 8, 4


# --------------------------------------------------------------------------------------------------- the fused node
class FusedElementwise:
    """``steps``: [(primitive name, [operand, ...])] with operands ("in", k), ("tmp", j) (result of step j) or
    ("const", number); ``outputs``: indices of the steps whose values leave the cluster."""

    def __init__(self, steps, outputs, n_inputs, dtype):
        self.steps, self.outputs, self.n_inputs, self.dtype = list(steps), list(outputs), n_inputs, dtype
        self.__name__ = "FusedElementwise"
        self.name = "FusedElementwise[%s]" % "+".join(s[0] for s in self.steps)
        self._lib = None

    # -- the expression with torch: CPU tensors, backward, and the oracle of the tests
    def reference(self, *inputs):
        vals = []
        ins = [t.float() for t in inputs]

        def get(ref):
            kind, v = ref
            return ins[v] if kind == "in" else vals[v] if kind == "tmp" else v
        for op, refs in self.steps:
            if op in _UNARY:
                vals.append(_UNARY[op][1](get(refs[0])))
            else:
                a, b = get(refs[0]), get(refs[1])
                if not isinstance(a, torch.Tensor):
                    a = torch.full_like(b, float(a))
                if op in ("Maximum", "Minimum") and not isinstance(b, torch.Tensor):
                    b = torch.full_like(a, float(b))
                vals.append(_BINARY[op][1](a, b))
        outs = tuple(vals[k].to(self.dtype) for k in self.outputs)
        return outs[0] if len(outs) == 1 else outs

    def __call__(self, *inputs):
        plain = [t.as_subclass(torch.Tensor) for t in inputs]
        if plain[0].is_cuda and all(t.is_contiguous() and t.dtype == self.dtype for t in plain):
            out = _FusedFn.apply(self, *plain)
            return out[0] if len(self.outputs) == 1 else out
        return self.reference(*plain)

    # -- the generated kernel
    def source(self):
        return kernel_source(self.steps, self.outputs, self.n_inputs, self.dtype)

    def launch(self, inputs):
        if self._lib is None:
            self._lib = _load(self.source())
        outs = [torch.empty_like(inputs[0]) for _ in self.outputs]
        n = inputs[0].numel()
        if n:
            ins_p = (ctypes.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
            outs_p = (ctypes.c_void_p * len(outs))(*[t.data_ptr() for t in outs])
            rc = self._lib.msb_gk_launch(ins_p, outs_p, ctypes.c_longlong(n),
                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            if rc != 0:
                raise RuntimeError("the generated kernel %s failed to launch (CUDA error %d)" % (self.name, rc))
        return tuple(outs)


class _FusedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, node, *inputs):
        ctx.node = node
        ctx.save_for_backward(*inputs)
        return node.launch(inputs)

    @staticmethod
    def backward(ctx, *grads):
        inputs = [t.detach().requires_grad_(True) for t in ctx.saved_tensors]
        with torch.enable_grad():
            outs = ctx.node.reference(*inputs)
            outs = outs if isinstance(outs, tuple) else (outs,)
            pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
            got = torch.autograd.grad([o for o, _ in pairs], inputs, [g for _, g in pairs], allow_unused=True) \
                if pairs else [None] * len(inputs)
        return (None,) + tuple(got)


def _literal(v):
    v = float(v)
    if v != v:
        return "__int_as_float(0x7fc00000)"
    if v in (float("inf"), float("-inf")):
        return "(%s__int_as_float(0x7f800000))" % ("-" if v < 0 else "")
    return "%sf" % repr(v) if ("." in repr(v) or "e" in repr(v)) else "%s.f" % repr(v)


def kernel_source(steps, outputs, n_inputs, dtype):
    """CUDA text of the kernel and of its host launcher ``msb_gk_launch(ins, outs, n, stream)``."""
    ctype, vec = _DTYPES[dtype]
    to_f = {"float": "%s", "__nv_bfloat16": "__bfloat162float(%s)", "__half": "__half2float(%s)"}[ctype]
    from_f = {"float": "%s", "__nv_bfloat16": "__float2bfloat16_rn(%s)", "__half": "__float2half_rn(%s)"}[ctype]

    def body(load, store, indent):
        lines = ["float x%d = %s;" % (k, to_f % load(k)) for k in range(n_inputs)]
        for j, (op, refs) in enumerate(steps):
            names = ["x%d" % v if kind == "in" else "t%d" % v if kind == "tmp" else "(%s)" % _literal(v)
                     for kind, v in refs]
            expr = _UNARY[op][0] if op in _UNARY else _BINARY[op][0]
            # substitute operands by token, not by character: the expressions call functions with a / b inside
            out = []
            for tok in _tokens(expr):
                out.append(names[0] if tok == "a" else names[1] if tok == "b" and len(names) > 1 else tok)
            lines.append("float t%d = %s;" % (j, "".join(out)))
        lines += [store(k, from_f % ("t%d" % o)) for k, o in enumerate(outputs)]
        return "\n".join(indent + ln for ln in lines)

    params = ", ".join(["const T* __restrict__ in%d" % k for k in range(n_inputs)] +
                       ["T* __restrict__ out%d" % k for k in range(len(outputs))])
    n_out = len(outputs)
    vec_params = ", ".join(["const V& vi%d" % k for k in range(n_inputs)] + ["V& vo%d" % k for k in range(n_out)])
    vec_body = body(lambda k: "vi%d.e[j]" % k, lambda k, v: "vo%d.e[j] = %s;" % (k, v), "        ")

    def vec_block(tag, at, indent):
        """Loads of one vector position, the call of the expression, the stores."""
        loads = ["V %si%d = reinterpret_cast<const V*>(in%d)[%s];" % (tag, k, k, at) for k in range(n_inputs)]
        call = ["V %s;" % ", ".join("%so%d" % (tag, k) for k in range(n_out)),
                "gk_vec(%s);" % ", ".join(["%si%d" % (tag, k) for k in range(n_inputs)] +
                                          ["%so%d" % (tag, k) for k in range(n_out)])]
        stores = ["reinterpret_cast<V*>(out%d)[%s] = %so%d;" % (k, at, tag, k) for k in range(n_out)]
        return ["\n".join(indent + ln for ln in part) for part in (loads, call + stores)]
    first_loads, first_rest = vec_block("a", "i", "        ")
    second_loads, second_rest = vec_block("b", "k", "            ")
    tail_body = body(lambda k: "in%d[i]" % k, lambda k, v: "out%d[i] = %s;" % (k, v), "        ")
    args = ", ".join(["(const T*)ins[%d]" % k for k in range(n_inputs)] +
                     ["(T*)outs[%d]" % k for k in range(len(outputs))])
    align = " | ".join(["(unsigned long long)ins[%d]" % k for k in range(n_inputs)] +
                       ["(unsigned long long)outs[%d]" % k for k in range(len(outputs))])
    return """#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
typedef %(ctype)s T;
struct __align__(16) V { T e[%(vec)d]; };

__device__ __forceinline__ void gk_vec(%(vec_params)s) {
#pragma unroll
    for (int j = 0; j < %(vec)d; ++j) {
%(vec_body)s
    }
}

// two 16-byte vectors per thread and iteration (both sets of loads are issued before the arithmetic: the kernel is
// bound by memory latency); the last n %% %(vec)d elements go through the scalar tail
__global__ void __launch_bounds__(256) gk_kernel(%(params)s, long long n_vec, long long n) {
    long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += 2 * stride) {
        long long k = i + stride;
%(first_loads)s
        if (k < n_vec) {
%(second_loads)s
%(second_rest)s
        }
%(first_rest)s
    }
    for (long long i = n_vec * %(vec)d + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
%(tail_body)s
    }
}

extern "C" __attribute__((visibility("default")))
int msb_gk_launch(void** ins, void** outs, long long n, void* stream) {
    // unaligned operands (a view into a larger buffer) take the scalar path for every element
    long long n_vec = ((%(align)s) & 15ull) ? 0 : n / %(vec)d;
    long long work = n_vec > 0 ? (n_vec + 1) / 2 : n;
    long long blocks = (work + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    gk_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(%(args)s, n_vec, n);
    return (int)cudaGetLastError();
}
""" % {"ctype": ctype, "vec": vec, "params": params, "vec_params": vec_params, "vec_body": vec_body,
       "first_loads": first_loads, "first_rest": first_rest, "second_loads": second_loads,
       "second_rest": second_rest, "tail_body": tail_body, "args": args, "align": align}


def _tokens(expr):
    """Splits a C expression into identifiers / numbers and the characters between them."""
    out, cur = [], ""
    for ch in expr:
        if ch.isalnum() or ch in "._":
            cur += ch
        else:
            if cur:
                out.append(cur)
                cur = ""
            out.append(ch)
    if cur:
        out.append(cur)
    return out


def _cache_dir():
    d = os.environ.get("MSB200_KERNEL_CACHE") or os.path.join(os.path.expanduser("~"), ".cache", "mindspore_b200",
                                                                 "graph_kernel")
    os.makedirs(d, exist_ok=True)
    return d


def compile_source(src, load=True):
    """nvcc -> shared object named by the hash of the source; returns the path (and loads nothing itself)."""
    from .._native.build import _nvcc
    digest = hashlib.sha256(src.encode()).hexdigest()[:24]
    lib = os.path.join(_cache_dir(), "gk_%s.so" % digest)
    if not os.path.exists(lib):
        cu = os.path.join(_cache_dir(), "gk_%s.cu" % digest)
        with open(cu, "w") as f:
            f.write(src)
        tmp = "%s.%d.tmp" % (lib, os.getpid())
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
               "-Xcompiler", "-fPIC", "-o", tmp, cu]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed for a generated kernel:\n%s\n%s" % (res.stderr[-2000:], src))
        os.replace(tmp, lib)                      # atomic: ranks compiling the same kernel do not collide
    return lib


def _load(src):
    lib = ctypes.CDLL(compile_source(src))
    lib.msb_gk_launch.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
    lib.msb_gk_launch.restype = ctypes.c_int
    return lib


# --------------------------------------------------------------------------------------------------- the pass
def _fusable(n):
    import torch.fx as fx
    if n.op != "call_function" or n.kwargs or not (hasattr(n.target, "name") and hasattr(n.target, "attrs")):
        return False
    op = n.target.name
    arity = 1 if op in _UNARY else 2 if op in _BINARY else 0
    if arity == 0 or len(n.args) != arity or n.meta.get("dtype") not in _DTYPES or "shape" not in n.meta:
        return False
    if getattr(n.target, "in_strategy", None) is not None:
        return False                                 # a sharded primitive goes through the SPMD dispatcher
    if n.meta.get("requires_vjp"):
        return False                                 # gradient nodes refer to this node by name: leave it
    tensors = 0
    for a in n.args:
        if isinstance(a, fx.Node):
            if tuple(a.meta.get("shape", ())) != tuple(n.meta["shape"]) or a.meta.get("dtype") != n.meta["dtype"]:
                return False
            tensors += 1
        elif isinstance(a, bool) or not isinstance(a, (int, float)):
            return False
    return tensors > 0


def fuse_elementwise(fg):
    """Replaces clusters of elementwise primitives by ``FusedElementwise`` nodes; returns the number of clusters."""
    import torch.fx as fx
    nodes = list(fg.graph.nodes)
    pos = {n: i for i, n in enumerate(nodes)}
    group_of, groups = {}, []

    def externally_used_before(members, limit, ignore):
        for m in members:
            for u in m.users:
                if u not in members and u is not ignore and pos[u] < limit:
                    return True
        return False

    def n_inputs(members):
        seen = set()
        for m in members:
            for a in m.args:
                if isinstance(a, fx.Node) and a not in members:
                    seen.add(a)
        return len(seen)

    for n in nodes:
        if not _fusable(n):
            continue
        merged = {n}
        for a in n.args:
            g = group_of.get(a) if isinstance(a, fx.Node) else None
            if g is None or groups[g] is None or groups[g] <= merged:
                continue
            trial = merged | groups[g]
            if len(trial) > MAX_NODES or n_inputs(trial) > MAX_INPUTS:
                continue
            if externally_used_before(trial, pos[n], n):
                continue
            merged = trial
        gid = len(groups)
        for m in merged:
            old = group_of.get(m)
            if old is not None:
                groups[old] = None
            group_of[m] = gid
        groups.append(merged)

    made = 0
    for members in groups:
        if members is None or len(members) < 2:
            continue
        ordered = sorted(members, key=pos.get)
        outs = [m for m in ordered if any(u not in members for u in m.users)]
        if not outs or len(outs) > MAX_OUTPUTS:
            continue
        inputs, steps, index = [], [], {}
        for m in ordered:
            refs = []
            for a in m.args:
                if isinstance(a, fx.Node):
                    if a in members:
                        refs.append(("tmp", index[a]))
                    else:
                        if a not in inputs:
                            inputs.append(a)
                        refs.append(("in", inputs.index(a)))
                else:
                    refs.append(("const", float(a)))
            index[m] = len(steps)
            steps.append((m.target.name, refs))
        last = ordered[-1]
        fused = FusedElementwise(steps, [index[m] for m in outs], len(inputs), last.meta["dtype"])
        with fg.graph.inserting_after(last):
            node = fg.graph.create_node("call_function", fused, tuple(inputs), {})
        node.meta.update({"shape": last.meta["shape"], "dtype": last.meta["dtype"], "primitive": "FusedElementwise"})
        if len(outs) == 1:
            outs[0].replace_all_uses_with(node)
        else:
            import operator
            anchor = node
            for k, m in enumerate(outs):
                with fg.graph.inserting_after(anchor):
                    item = fg.graph.create_node("call_function", operator.getitem, (node, k), {})
                item.meta.update({"shape": m.meta["shape"], "dtype": m.meta["dtype"]})
                m.replace_all_uses_with(item)
                anchor = item
        for m in reversed(ordered):
            fg.graph.erase_node(m)
        made += 1
    if made:
        fg.graph.lint()
    return made


def _bench(n=1 << 27, iters=10):
    """Times one six-primitive cluster (2 inputs, 2 outputs, bf16, tensors larger than L2) as the generated kernel and
    as six separate torch operators; prints one JSON line with the achieved bandwidth of each."""
    import json
    steps = [("Add", [("in", 0), ("in", 1)]), ("Mul", [("tmp", 0), ("const", 2.0)]), ("Tanh", [("tmp", 1)]),
             ("Sub", [("const", 1.5), ("tmp", 2)]), ("Maximum", [("tmp", 3), ("in", 0)]), ("ReLU", [("tmp", 0)])]
    fused = FusedElementwise(steps, [4, 5], 2, torch.bfloat16)
    x = torch.randn(n, device="cuda").to(torch.bfloat16)
    y = torch.randn(n, device="cuda").to(torch.bfloat16)

    def unfused():
        a = x + y
        return torch.maximum(1.5 - torch.tanh(a * 2.0), x), torch.relu(a)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / iters

    with torch.no_grad():
        t_fused = timed(lambda: fused.launch((x, y)))
        t_plain = timed(unfused)
        got, want = fused.launch((x, y)), unfused()
    err = max(float((g.float() - w.float()).abs().max()) for g, w in zip(got, want))
    algorithmic = 4 * n * 2                                    # two inputs read, two outputs written
    print(json.dumps({"kernel": fused.name, "elements": n, "dtype": "bf16", "fused_ms": round(t_fused, 4),
                      "unfused_ms": round(t_plain, 4), "fused_gbs": round(algorithmic / t_fused / 1e6, 1),
                      "speedup": round(t_plain / t_fused, 2), "max_abs_diff_vs_unfused": err}))


if __name__ == "__main__":
    _bench()

"""``Profiler``: device and host timeline of a training run.

    prof = Profiler(output_path="./prof", profile_memory=False, start_profile=True)
    ... training steps ...
    prof.stop(); prof.analyse()

``analyse`` writes, under ``<output_path>/profiler/``: ``kernel_time_<rank>.csv`` (every GPU kernel aggregated by
name: calls, total / mean microseconds, share), ``op_type_<rank>.csv`` (framework-level operators), a Chrome-trace
``timeline_<rank>.json`` and, with ``profile_memory``, ``memory_<rank>.csv``; ``op_analyse`` returns the kernel table
as a list of dicts.  The collection itself is CUPTI through ``torch.profiler`` (the reference drives CUPTI directly:
plugin/device/gpu/hal/profiler/gpu_profiling.cc, cupti_interface.cc; Python side profiler/profiling.py:340-1036).
Environment switch like the reference's ``MS_PROFILER_OPTIONS``: a JSON object with ``start`` / ``output_path``
makes ``EnvProfiler.from_env()`` return a started profiler.

``python -m mindspore_b200.profiler --model resnet50|llama --steps N`` profiles a few steps of a built-in model and
prints the kernel table (the command behind the summaries in ``profiles/``)."""
from __future__ import annotations

import csv
import json
import os
import sys
import time

import torch


class ProfilerLevel:
    """How much the profiler collects (python/mindspore/profiler/common/constant.py): Level0 - step and collective
    ranges only, Level1 - plus kernel tables, Level2 - plus memory and call stacks."""
    Level0 = "Level0"
    Level1 = "Level1"
    Level2 = "Level2"


class Profiler:
    def __init__(self, output_path="./data", profile_communication=False, profile_memory=False, op_time=True,
                 data_process=False, timeline_limit=500, start_profile=True, l2_cache=False, with_stack=False, **kw):
        self.output_path = os.path.join(os.path.abspath(output_path), "profiler")
        self.profile_memory, self.op_time, self.with_stack = profile_memory, op_time, with_stack
        self.profile_communication = profile_communication
        self.timeline_limit = timeline_limit
        self._prof = None
        self._t0 = self._t1 = None
        self.rank = int(os.environ.get("RANK", os.environ.get("RANK_ID", "0")))
        if start_profile:
            self.start()

    def start(self):
        if self._prof is not None:
            raise RuntimeError("The profiler has already started.")
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, profile_memory=self.profile_memory,
                                            with_stack=self.with_stack, record_shapes=False)
        self._prof.__enter__()
        _active[0] += 1
        self._t0 = time.time()

    def stop(self):
        if self._prof is None:
            raise RuntimeError("The profiler has not started.")
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self._prof.__exit__(None, None, None)
        _active[0] = max(0, _active[0] - 1)
        self._t1 = time.time()

    # ------------------------------------------------------------------ analysis
    def _events(self):
        if self._prof is None or self._t1 is None:
            raise RuntimeError("call stop() before analysing")
        return self._prof.events()

    def op_analyse(self, op_name=None, device_id=None):
        """[{name, calls, total_us, mean_us, share}] of device kernels, longest first."""
        agg = {}
        for e in self._events():
            if e.device_type != torch.autograd.DeviceType.CUDA:
                continue
            name = e.name
            if op_name and op_name not in name:
                continue
            a = agg.setdefault(name, [0, 0.0])
            a[0] += 1
            a[1] += e.device_time if hasattr(e, "device_time") else e.cuda_time
        total = sum(v[1] for v in agg.values()) or 1.0
        rows = [{"name": k, "calls": v[0], "total_us": round(v[1], 1), "mean_us": round(v[1] / v[0], 2),
                 "share": round(v[1] / total, 4)} for k, v in agg.items()]
        return sorted(rows, key=lambda r: -r["total_us"])

    @classmethod
    def offline_analyse(cls, path, pretty=False, step_list=None, data_simplification=True):
        """Re-reads what a finished run wrote under ``path`` (``kernel_time_<rank>.csv``) and returns the kernel
        rows per rank: nothing is re-collected."""
        out = {}
        for name in sorted(os.listdir(path)):
            if name.startswith("kernel_time_") and name.endswith(".csv"):
                with open(os.path.join(path, name), newline="") as f:
                    out[int(name[len("kernel_time_"):-4])] = list(csv.DictReader(f))
        if not out:
            raise RuntimeError("offline_analyse: no kernel_time_<rank>.csv under %s" % path)
        return out

    def analyse(self, offline_path=None, pretty=False, step_list=None, mode="sync"):
        os.makedirs(self.output_path, exist_ok=True)
        kernels = self.op_analyse()
        with open(os.path.join(self.output_path, "kernel_time_%d.csv" % self.rank), "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=["name", "calls", "total_us", "mean_us", "share"])
            w.writeheader()
            w.writerows(kernels)
        host = {}
        for e in self._events():
            if e.device_type == torch.autograd.DeviceType.CPU:
                a = host.setdefault(e.name, [0, 0.0])
                a[0] += 1
                a[1] += e.cpu_time_total
        with open(os.path.join(self.output_path, "op_type_%d.csv" % self.rank), "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["op_type", "calls", "host_total_us"])
            for k, v in sorted(host.items(), key=lambda kv: -kv[1][1]):
                w.writerow([k, v[0], round(v[1], 1)])
        self._prof.export_chrome_trace(os.path.join(self.output_path, "timeline_%d.json" % self.rank))
        trace = self.step_trace()
        if trace:
            with open(os.path.join(self.output_path, "step_trace_%d.csv" % self.rank), "w", newline="") as f:
                w = csv.DictWriter(f, fieldnames=list(trace[0]))
                w.writeheader()
                w.writerows(trace)
        if self.profile_memory:
            with open(os.path.join(self.output_path, "memory_%d.csv" % self.rank), "w", newline="") as f:
                w = csv.writer(f)
                w.writerow(["name", "self_device_memory_bytes", "self_cpu_memory_bytes"])
                for e in self._prof.key_averages():
                    w.writerow([e.key, getattr(e, "self_device_memory_usage", 0), e.self_cpu_memory_usage])
        return kernels

    # ------------------------------------------------------------------ step trace
    COMM = ("nccl", "symm_barrier", "allreduce_symm", "reduce_slots", "reduce_scatter_symm", "all_gather", "Memcpy PtoP",
            "moe_dispatch", "moe_combine")
    OPT = ("adamw", "momentum_kernel", "sumsq_finite", "finalize_grad_scale", "multi_tensor", "FusedAdam", "fused_sgd")
    BWD = ("bwd", "dgrad", "wgrad", "_grad", "Backward", "backward")

    @classmethod
    def classify(cls, name):
        """forward / backward / optimizer / comm for a device kernel name.  The GEMM's role follows its operand
        layouts (template flags of ``gemm_bf16_kernel<BN, A_MN, B_MN, MODE>`` / ``gemm2_bf16_kernel<A_MN, B_MN, ..>``):
        B stored [K, N] is a dgrad, both operands MN-major a wgrad; MODE 1 / 2 carry their collective inside."""
        low = name
        if any(k in low for k in cls.COMM):
            return "comm"
        if any(k in low for k in cls.OPT):
            return "optimizer"
        if "gemm_bf16_kernel<" in low or "gemm2_bf16_kernel<" in low:
            flags = low.split("<", 1)[1].split(">")[0].replace(" ", "").split(",")
            bools = [f for f in flags if f in ("true", "false")]
            if len(bools) >= 2 and bools[1] == "true":
                return "backward"
            return "forward"
        if any(k in low for k in cls.BWD):
            return "backward"
        return "forward"

    def step_trace(self):
        """Per training step (``msb::step`` ranges recorded by the train-step cells; the whole capture when there are
        none): device time by phase, the part of communication not hidden behind compute, and idle gaps - the
        split of the reference's step trace (profiler/parser/step_trace_parser.py: iteration interval, fp_and_bp,
        tail; gpu_profiling.cc:459-547 for the kernel / op correlation)."""
        evs = list(self._events())
        kernels = sorted(((e.time_range.start, e.time_range.end, e.name) for e in evs
                          if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda k: k[0])
        steps = sorted((e.time_range.start, e.time_range.end) for e in evs
                       if e.device_type == torch.autograd.DeviceType.CPU and e.name == "msb::step")
        if not kernels:
            return []
        if not steps:
            windows = [(kernels[0][0], max(k[1] for k in kernels))]
        else:
            # a step's kernels run after its CPU range starts and before the next step's first kernel
            windows = []
            for i, (s0, s1) in enumerate(steps):
                nxt = steps[i + 1][0] if i + 1 < len(steps) else float("inf")
                ks = [k for k in kernels if s0 <= k[0] < nxt]
                if ks:
                    windows.append((ks[0][0], max(k[1] for k in ks)))
        rows = []
        for i, (w0, w1) in enumerate(windows):
            ks = [k for k in kernels if w0 <= k[0] <= w1]
            by = {"forward": 0.0, "backward": 0.0, "optimizer": 0.0, "comm": 0.0}
            marks = []
            for a, b, name in ks:
                c = self.classify(name)
                by[c] += b - a
                marks.append((a, 1, c == "comm"))
                marks.append((b, -1, c == "comm"))
            marks.sort(key=lambda m: (m[0], m[1]))
            busy = exposed = 0.0
            n_all = n_comm = 0
            prev = None
            for t, d, is_comm in marks:
                if prev is not None and n_all > 0:
                    busy += t - prev
                    if n_comm == n_all:
                        exposed += t - prev
                n_all += d
                if is_comm:
                    n_comm += d
                prev = t
            total = w1 - w0
            rows.append({"step": i, "total_ms": round(total / 1e3, 3), "fp_ms": round(by["forward"] / 1e3, 3),
                         "bp_ms": round(by["backward"] / 1e3, 3), "optimizer_ms": round(by["optimizer"] / 1e3, 3),
                         "comm_ms": round(by["comm"] / 1e3, 3), "comm_exposed_ms": round(exposed / 1e3, 3),
                         "gap_ms": round((total - busy) / 1e3, 3), "kernels": len(ks)})
        return rows

    def summary(self, top=30):
        rows = self.op_analyse()
        total = sum(r["total_us"] for r in rows)
        lines = ["device time %.3f ms over %.3f s wall" % (total / 1000, (self._t1 or 0) - (self._t0 or 0))]
        for r in rows[:top]:
            lines.append("%10.3f ms %6.2f%% n=%5d  %s" % (r["total_us"] / 1000, 100 * r["share"], r["calls"],
                                                         r["name"][:110]))
        return "\n".join(lines)


_active = [0]


def step_range():
    """Context manager the train-step cells wrap one step in: a ``msb::step`` range when a profiler is running."""
    if _active[0] > 0:
        return torch.profiler.record_function("msb::step")
    import contextlib
    return contextlib.nullcontext()


class EnvProfiler:
    """Profiler configured by ``MS_PROFILER_OPTIONS`` (JSON: start, output_path, profile_memory, ...)."""

    @staticmethod
    def from_env():
        raw = os.environ.get("MS_PROFILER_OPTIONS")
        if not raw:
            return None
        try:
            opt = json.loads(raw)
        except ValueError as e:
            raise ValueError("MS_PROFILER_OPTIONS is not valid JSON: %s" % e)
        if not opt.get("start", False):
            return None
        return Profiler(output_path=opt.get("output_path", "./data"), profile_memory=opt.get("profile_memory", False),
                        start_profile=True)


def _main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(prog="mindspore_b200.profiler")
    ap.add_argument("--model", choices=["resnet50", "llama"], default="resnet50")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--layers", type=int, default=4, help="llama: number of layers (7B shapes)")
    ap.add_argument("--out", default="./profiler_out")
    args = ap.parse_args(argv)
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    ms.set_context(device_target="GPU")
    ms.set_seed(0)
    if args.model == "resnet50":
        from mindspore_b200.models.resnet import ResNetWithLoss, resnet50
        net = ResNetWithLoss(resnet50(1000, dtype=torch.bfloat16))
        opt = nn.Momentum(net.trainable_params(), 0.1, 0.9, weight_decay=1e-4)
        inputs = (ms.Tensor(torch.randn(args.batch, 3, 224, 224, device="cuda").bfloat16()),
                  ms.Tensor(torch.randint(0, 1000, (args.batch,), device="cuda")))
    else:
        from mindspore_b200.models.llama import LlamaConfig, LlamaForCausalLM
        cfg = LlamaConfig()
        cfg.num_layers = args.layers
        net = LlamaForCausalLM(cfg)
        opt = nn.AdamWeightDecay(net.trainable_params(), learning_rate=1e-4, max_grad_norm=1.0)
        inputs = (ms.Tensor(torch.randint(0, cfg.vocab_size, (1, cfg.seq_length + 1), dtype=torch.int32,
                                          device="cuda")),)
    step = nn.TrainOneStepCell(net, opt)
    step.set_train()
    for _ in range(2):
        step(*inputs)
    prof = Profiler(output_path=args.out)
    for _ in range(args.steps):
        step(*inputs)
    prof.stop()
    prof.analyse()
    print(prof.summary(40))
    for row in prof.step_trace():
        print("step %(step)d: %(total_ms).2f ms = fp %(fp_ms).2f + bp %(bp_ms).2f + optimizer %(optimizer_ms).2f + "
              "comm %(comm_ms).2f (exposed %(comm_exposed_ms).2f) + gaps %(gap_ms).2f" % row)
    return 0


if __name__ == "__main__":
    sys.exit(_main())

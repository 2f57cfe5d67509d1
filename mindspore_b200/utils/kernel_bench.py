"""Micro-benchmarks of the sm_100a kernels: ``python -m mindspore_b200.utils.kernel_bench <what> [options]``.

Each benchmark warms up, then times at least ``--iters`` launches - and at least ``--min-ms`` of device time, so that
the 200 ms clock sampler sees the region - with CUDA events on the launching stream.  Between timed launches the
operands rotate through enough distinct buffers to exceed the L2 capacity (``--l2-mb``), so every launch reads its
inputs from HBM.  One JSON line per case goes to stdout; every row carries the SM clock sampled during its timed
region (``sm_mhz``: median under load, ``sm_max_mhz``, throttle ``reasons``) and ``ms_x_mhz`` (time x clock, the
quantity to compare between runs that saw different clocks).  A row whose reasons include a hardware or thermal
slowdown is not a valid performance number.  With ``--once`` a case is launched a few times without timing (the form
to run under a profiler on a small problem)."""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch


_sampler = None
_min_ms = 1500.0
_last_clocks = {}


def _time(fn, sets, iters, warmup=3):
    """Mean milliseconds per launch; the clocks seen during the timed region are left in ``_last_clocks``."""
    import time
    for i in range(warmup):
        fn(*sets[i % len(sets)])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(3):
        fn(*sets[i % len(sets)])
    e1.record()
    torch.cuda.synchronize()
    est = max(e0.elapsed_time(e1) / 3, 1e-3)
    iters = max(iters, int(math.ceil(_min_ms / est)))
    t0 = time.time()
    e0.record()
    for i in range(iters):
        fn(*sets[i % len(sets)])
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ms = e0.elapsed_time(e1) / iters
    _last_clocks.clear()
    if _sampler is not None:
        time.sleep(0.25)                      # let the sample that covers the end of the region arrive
        _last_clocks.update(_sampler.window(t0, t1))
        _last_clocks["iters"] = iters
    return ms


def _clk(ms, prefix=""):
    c = dict(_last_clocks)
    out = {prefix + "sm_mhz": c.get("sm_mhz"), prefix + "reasons": c.get("reasons")}
    if not prefix:
        out["sm_max_mhz"] = c.get("sm_max_mhz")
    if c.get("sm_mhz"):
        out[prefix + "ms_x_mhz"] = round(ms * c["sm_mhz"], 2)
    return out


def _nsets(bytes_per_set, l2_mb):
    return max(2, int(math.ceil(l2_mb * 2 ** 20 / max(bytes_per_set, 1))) + 1)


def _emit(**kw):
    print(json.dumps(kw), flush=True)


def bench_gemm(args):
    from ..ops import kernels as K
    for spec in args.shapes or ["4096x4096x4096", "8192x8192x8192", "4096x22016x4096", "4096x4096x11008"]:
        M, N, Kd = (int(v) for v in spec.split("x"))
        for a_mn, b_mn in ((False, False), (False, True), (True, True)):
            if args.layout and args.layout != "%d%d" % (a_mn, b_mn):
                continue
            n = _nsets((M * Kd + N * Kd + M * N) * 2, args.l2_mb)
            sets = [(torch.randn((Kd, M) if a_mn else (M, Kd), device="cuda").bfloat16(),
                     torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda").bfloat16(),
                     torch.empty(M, N, device="cuda", dtype=torch.bfloat16)) for _ in range(n)]
            ours = lambda a, b, c: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=c, bn_hint=args.bn)
            if args.once:
                for s in sets[:3]:
                    ours(*s)
                torch.cuda.synchronize()
                continue
            lib = lambda a, b, c: torch.matmul(a.t() if a_mn else a, b if b_mn else b.t(), out=c)
            ms = _time(ours, sets, args.iters)
            c_ours = _clk(ms)
            ms_lib = _time(lib, sets, args.iters)
            c_lib = _clk(ms_lib, "cublas_")
            fl = 2.0 * M * N * Kd
            _emit(kernel="gemm_bf16", M=M, N=N, K=Kd, a_mn=a_mn, b_mn=b_mn, ms=round(ms, 4),
                  tflops=round(fl / ms / 1e9, 1), cublas_ms=round(ms_lib, 4), cublas_tflops=round(fl / ms_lib / 1e9, 1),
                  buffers=n, **c_ours, **c_lib)


def bench_attention(args):
    from ..ops import flash_attn_kernel as FK
    D = 128
    for S in args.seq or [4096]:
        for causal in (True, False):
            B, H = args.batch, args.heads
            n = _nsets(4 * B * S * H * D * 2, args.l2_mb)
            sets = [tuple(torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(4)) for _ in range(n)]
            sc = 1 / math.sqrt(D)
            fwd = lambda q, k, v, do: FK.fwd(q, k, v, causal, sc)
            if args.once:
                for s in sets[:2]:
                    o, lse, q2, k2, v2 = fwd(*s)
                    FK.bwd(s[3], q2, k2, v2, o, lse, causal, sc)
                torch.cuda.synchronize()
                continue
            outs = [fwd(*s) for s in sets]
            bwd_sets = [(s[3], o[2], o[3], o[4], o[0], o[1]) for s, o in zip(sets, outs)]
            bwd = lambda do, q, k, v, o, lse: FK.bwd(do, q, k, v, o, lse, causal, sc)
            ms_f = _time(fwd, sets, args.iters)
            c_f = _clk(ms_f, "fwd_")
            ms_b = _time(bwd, bwd_sets, args.iters)
            c_b = _clk(ms_b, "bwd_")
            lib_sets = [tuple(t.permute(0, 2, 1, 3).detach().requires_grad_(True) for t in s[:3]) + (s[3].permute(0, 2, 1, 3),)
                        for s in sets]
            sdpa = torch.nn.functional.scaled_dot_product_attention
            lib_f = lambda q, k, v, do: sdpa(q, k, v, is_causal=causal)
            lib_outs = [lib_f(*s) for s in lib_sets]
            lib_b_sets = [(o, s) for o, s in zip(lib_outs, lib_sets)]
            lib_b = lambda o, s: torch.autograd.grad(o, s[:3], s[3], retain_graph=True)
            ms_lf = _time(lib_f, lib_sets, args.iters)
            c_lf = _clk(ms_lf, "sdpa_fwd_")
            ms_lb = _time(lib_b, lib_b_sets, args.iters)
            c_lb = _clk(ms_lb, "sdpa_bwd_")
            f = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
            _emit(kernel="flash_attention", B=B, S=S, H=H, D=D, causal=causal, fwd_ms=round(ms_f, 4),
                  fwd_tflops=round(f / ms_f / 1e9, 1), bwd_ms=round(ms_b, 4), bwd_tflops=round(2.5 * f / ms_b / 1e9, 1),
                  sdpa_fwd_ms=round(ms_lf, 4), sdpa_fwd_tflops=round(f / ms_lf / 1e9, 1), sdpa_bwd_ms=round(ms_lb, 4),
                  sdpa_bwd_tflops=round(2.5 * f / ms_lb / 1e9, 1), buffers=n, **c_f, **c_b, **c_lf, **c_lb)


def bench_elementwise(args):
    """Memory-bound kernels: achieved GB/s over algorithmic bytes."""
    from ..ops import kernels as K
    rows, H, F = args.rows, 4096, 11008
    n = _nsets(rows * H * 2 * 4, args.l2_mb)
    mk = lambda *s: torch.randn(*s, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    sets = [(mk(rows, H), mk(rows, H)) for _ in range(n)]
    ms = _time(lambda x, r: K.rmsnorm_fwd(x, w, 1e-5, residual=r), sets, args.iters)
    _emit(kernel="rmsnorm_fwd+residual", rows=rows, H=H, ms=round(ms, 4), gbs=round(rows * H * 2 * 4 / ms / 1e6, 1), **_clk(ms))
    y, rstd, xs = K.rmsnorm_fwd(sets[0][0], w, 1e-5, residual=sets[0][1])
    ms = _time(lambda x, r: K.rmsnorm_bwd(x, r, w, rstd, dresidual=x), sets, args.iters)
    _emit(kernel="rmsnorm_bwd+dresidual", rows=rows, H=H, ms=round(ms, 4), gbs=round(rows * H * 2 * 4 / ms / 1e6, 1), **_clk(ms))
    n2 = _nsets(rows * F * 2 * 3, args.l2_mb)
    gsets = [(mk(rows, 2 * F), mk(rows, F)) for _ in range(n2)]
    ms = _time(lambda gu, do: K.swiglu_fwd(gu), gsets, args.iters)
    _emit(kernel="swiglu_fwd", rows=rows, F=F, ms=round(ms, 4), gbs=round(rows * F * 2 * 3 / ms / 1e6, 1), **_clk(ms))
    ms = _time(lambda gu, do: K.swiglu_bwd(gu, do), gsets, args.iters)
    _emit(kernel="swiglu_bwd", rows=rows, F=F, ms=round(ms, 4), gbs=round(rows * F * 2 * 5 / ms / 1e6, 1), **_clk(ms))
    nel = 1 << 28
    p, m, v, g = (torch.randn(nel, device="cuda") for _ in range(4))
    lp = torch.empty(nel, device="cuda", dtype=torch.bfloat16)
    hy = torch.tensor([1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0], device="cuda")
    ms = _time(lambda: K.adamw_step(p, m, v, g, lp, hy), [()], args.iters)
    _emit(kernel="adamw", n=nel, ms=round(ms, 4), gbs=round(nel * (4 * 7 + 2) / ms / 1e6, 1), **_clk(ms))


def bench_fused_comm(args):
    """The four model-parallel collective GEMMs of a Llama-2-7B layer (one micro-batch of 4096 tokens, mp = world
    size): fused NVLink kernel vs the same GEMM followed / preceded by the NCCL collective vs the GEMM alone.  Run
    under torchrun, one rank per GPU; every number is device time of calls replayed from one CUDA graph (no host
    launch time), max over ranks.  Also prints the roofline of each op: the slower of its FLOPs at the measured GEMM
    rate and its NVLink bytes at the measured per-direction peer bandwidth."""
    import json
    import torch.distributed as dist
    import mindspore_b200 as ms
    from ..communication import comm_func as CF
    from ..communication import init
    from ..communication import management as M
    from ..ops import fused
    from ..parallel import fused_comm as FC
    from ..parallel import tp as TP
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2:
        print("fused_comm needs torchrun with at least 2 ranks", file=sys.stderr)
        return
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    ms.set_context(device_target="GPU", device_id=local)
    init("nccl")
    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank,
                                 full_batch=True)
    tp, g = TP.TPGroup(), M._group(None)

    def timed(fn, iters=10, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(iters):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / (iters * reps)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del graph
        return t.item() * 1000.0                                     # microseconds

    peaks = {}
    try:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except (OSError, ValueError):
        pass
    tflops = float(peaks.get("bf16_tflops", 1590.0))
    link_gbs = 770.0                                                 # measured peer copy, per direction per GPU
    T, H, F = 4096, 4096, 11008
    bf = dict(device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        xs = torch.randn(T // world, H, **bf)
        wqkv, wgu = torch.randn(3 * H // world, H, **bf), torch.randn(2 * F // world, H, **bf)
        xo, wo = torch.randn(T, H // world, **bf), torch.randn(H, H // world, **bf)
        xd, wd = torch.randn(T, F // world, **bf), torch.randn(H, F // world, **bf)
        xf = torch.randn(T, H, **bf)
        cases = (
            ("allgather+qkv", (T, 3 * H // world, H), T * H * 2 * (world - 1) / world,
             lambda: FC.allgather_matmul(xs, wqkv, tp), lambda: fused.linear(CF._all_gather(xs, g), wqkv),
             lambda: fused.linear(xf, wqkv)),
            ("allgather+gate_up", (T, 2 * F // world, H), T * H * 2 * (world - 1) / world,
             lambda: FC.allgather_matmul(xs, wgu, tp), lambda: fused.linear(CF._all_gather(xs, g), wgu),
             lambda: fused.linear(xf, wgu)),
            ("wo+reducescatter", (T, H, H // world), T * H * 2 * (world - 1) / world,
             lambda: FC.matmul_reduce_scatter(xo, wo, tp), lambda: CF._reduce_scatter(fused.linear(xo, wo), "sum", g),
             lambda: fused.linear(xo, wo)),
            ("down+reducescatter", (T, H, F // world), T * H * 2 * (world - 1) / world,
             lambda: FC.matmul_reduce_scatter(xd, wd, tp), lambda: CF._reduce_scatter(fused.linear(xd, wd), "sum", g),
             lambda: fused.linear(xd, wd)))
        for name, (m, n, k), link_bytes, f_fused, f_nccl, f_gemm in cases:
            t_fused, t_nccl, t_gemm = timed(f_fused), timed(f_nccl), timed(f_gemm)
            t_math = 2.0 * m * n * k / (tflops * 1e12) * 1e6
            t_link = link_bytes / (link_gbs * 1e9) * 1e6
            roof = max(t_math, t_link)
            if rank == 0:
                _emit(kernel=name, world=world, m=m, n=n, k=k, fused_us=round(t_fused, 1),
                      gemm_plus_nccl_us=round(t_nccl, 1), gemm_alone_us=round(t_gemm, 1),
                      roofline_us=round(roof, 1), bound="link" if t_link > t_math else "math",
                      fused_of_roofline=round(roof / t_fused, 3))
    from .. import _native
    torch.cuda.synchronize()
    st = torch.tensor([_native.device_status()], device="cuda")
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    if rank == 0:
        _emit(device_status=int(st.item()))
    dist.barrier()
    M.release()


def main(argv=None):
    ap = argparse.ArgumentParser(prog="kernel_bench")
    ap.add_argument("what", choices=["gemm", "attention", "elementwise", "fused_comm"])
    ap.add_argument("--shapes", nargs="*", help="gemm: MxNxK ...")
    ap.add_argument("--layout", help="gemm: 00 (fwd), 01 (dgrad) or 11 (wgrad)")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--seq", nargs="*", type=int)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--l2-mb", type=int, default=128)
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--min-ms", type=float, default=1500.0, help="shortest timed region per case (clock sampling)")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("kernel_bench needs a CUDA device", file=sys.stderr)
        return 1
    if args.what == "fused_comm":
        bench_fused_comm(args)
        return 0
    global _sampler, _min_ms
    _min_ms = args.min_ms
    if not args.once:
        from .clocks import ClockSampler
        _sampler = ClockSampler(torch.cuda.current_device()).start()
    try:
        {"gemm": bench_gemm, "attention": bench_attention, "elementwise": bench_elementwise}[args.what](args)
    finally:
        if _sampler is not None:
            _sampler.stop()
    from .. import _native
    torch.cuda.synchronize()
    _emit(device_status=_native.device_status())
    return 0


if __name__ == "__main__":
    sys.exit(main())

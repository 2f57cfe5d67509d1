"""Micro-benchmarks of the sm_100a kernels: ``python -m mindspore_b200.utils.kernel_bench <what> [options]``.

Each benchmark warms up, then times ``--iters`` launches with CUDA events on the launching stream.  Between timed
launches the operands rotate through enough distinct buffers to exceed the L2 capacity (``--l2-mb``), so every launch
reads its inputs from HBM.  One JSON line per case goes to stdout.  With ``--once`` a case is launched a few times
without timing (the form to run under a profiler on a small problem)."""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch


def _time(fn, sets, iters, warmup=3):
    for i in range(warmup):
        fn(*sets[i % len(sets)])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(iters):
        fn(*sets[i % len(sets)])
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


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
            ms, ms_lib = _time(ours, sets, args.iters), _time(lib, sets, args.iters)
            fl = 2.0 * M * N * Kd
            _emit(kernel="gemm_bf16", M=M, N=N, K=Kd, a_mn=a_mn, b_mn=b_mn, ms=round(ms, 4),
                  tflops=round(fl / ms / 1e9, 1), cublas_ms=round(ms_lib, 4), cublas_tflops=round(fl / ms_lib / 1e9, 1),
                  buffers=n)


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
            ms_f, ms_b = _time(fwd, sets, args.iters), _time(bwd, bwd_sets, args.iters)
            lib_sets = [tuple(t.permute(0, 2, 1, 3).detach().requires_grad_(True) for t in s[:3]) + (s[3].permute(0, 2, 1, 3),)
                        for s in sets]
            sdpa = torch.nn.functional.scaled_dot_product_attention
            lib_f = lambda q, k, v, do: sdpa(q, k, v, is_causal=causal)
            lib_outs = [lib_f(*s) for s in lib_sets]
            lib_b_sets = [(o, s) for o, s in zip(lib_outs, lib_sets)]
            lib_b = lambda o, s: torch.autograd.grad(o, s[:3], s[3], retain_graph=True)
            ms_lf, ms_lb = _time(lib_f, lib_sets, args.iters), _time(lib_b, lib_b_sets, args.iters)
            f = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
            _emit(kernel="flash_attention", B=B, S=S, H=H, D=D, causal=causal, fwd_ms=round(ms_f, 4),
                  fwd_tflops=round(f / ms_f / 1e9, 1), bwd_ms=round(ms_b, 4), bwd_tflops=round(2.5 * f / ms_b / 1e9, 1),
                  sdpa_fwd_ms=round(ms_lf, 4), sdpa_fwd_tflops=round(f / ms_lf / 1e9, 1), sdpa_bwd_ms=round(ms_lb, 4),
                  sdpa_bwd_tflops=round(2.5 * f / ms_lb / 1e9, 1), buffers=n)


def bench_elementwise(args):
    """Memory-bound kernels: achieved GB/s over algorithmic bytes."""
    from ..ops import kernels as K
    rows, H, F = args.rows, 4096, 11008
    n = _nsets(rows * H * 2 * 4, args.l2_mb)
    mk = lambda *s: torch.randn(*s, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    sets = [(mk(rows, H), mk(rows, H)) for _ in range(n)]
    ms = _time(lambda x, r: K.rmsnorm_fwd(x, w, 1e-5, residual=r), sets, args.iters)
    _emit(kernel="rmsnorm_fwd+residual", rows=rows, H=H, ms=round(ms, 4), gbs=round(rows * H * 2 * 4 / ms / 1e6, 1))
    y, rstd, xs = K.rmsnorm_fwd(sets[0][0], w, 1e-5, residual=sets[0][1])
    ms = _time(lambda x, r: K.rmsnorm_bwd(x, r, w, rstd, dresidual=x), sets, args.iters)
    _emit(kernel="rmsnorm_bwd+dresidual", rows=rows, H=H, ms=round(ms, 4), gbs=round(rows * H * 2 * 4 / ms / 1e6, 1))
    n2 = _nsets(rows * F * 2 * 3, args.l2_mb)
    gsets = [(mk(rows, 2 * F), mk(rows, F)) for _ in range(n2)]
    ms = _time(lambda gu, do: K.swiglu_fwd(gu), gsets, args.iters)
    _emit(kernel="swiglu_fwd", rows=rows, F=F, ms=round(ms, 4), gbs=round(rows * F * 2 * 3 / ms / 1e6, 1))
    ms = _time(lambda gu, do: K.swiglu_bwd(gu, do), gsets, args.iters)
    _emit(kernel="swiglu_bwd", rows=rows, F=F, ms=round(ms, 4), gbs=round(rows * F * 2 * 5 / ms / 1e6, 1))
    nel = 1 << 28
    p, m, v, g = (torch.randn(nel, device="cuda") for _ in range(4))
    lp = torch.empty(nel, device="cuda", dtype=torch.bfloat16)
    hy = torch.tensor([1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0], device="cuda")
    ms = _time(lambda: K.adamw_step(p, m, v, g, lp, hy), [()], args.iters)
    _emit(kernel="adamw", n=nel, ms=round(ms, 4), gbs=round(nel * (4 * 7 + 2) / ms / 1e6, 1))


def main(argv=None):
    ap = argparse.ArgumentParser(prog="kernel_bench")
    ap.add_argument("what", choices=["gemm", "attention", "elementwise"])
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
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("kernel_bench needs a CUDA device", file=sys.stderr)
        return 1
    {"gemm": bench_gemm, "attention": bench_attention, "elementwise": bench_elementwise}[args.what](args)
    from .. import _native
    torch.cuda.synchronize()
    _emit(device_status=_native.device_status())
    return 0


if __name__ == "__main__":
    sys.exit(main())

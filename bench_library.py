"""Library baseline arm of ``bench.py`` (``--impl library``): the same models, configs, batch sizes and parallel
strategies written on stock PyTorch only - GEMMs through cuBLAS (``F.linear``), attention through
``F.scaled_dot_product_attention``, convolutions / batch norm through cuDNN, ``torch.optim`` fused optimizers, and every
collective a separate NCCL call (``all_gather_into_tensor`` / ``reduce_scatter_tensor`` / ``all_reduce``; the
data-parallel gradient all-reduce is ``DistributedDataParallel`` with 25 MB buckets on its own stream).  Nothing of
``mindspore_b200`` is imported here: no kernel, no engine, no collective of this repository is on this path.

It stands in for "the reference's execution model on the same box": per-operator library kernels plus un-fused
NCCL collectives (the reference's GPU build itself cannot be installed offline).  It is named *library*, never
*reference*.  Micro-batches are replayed as CUDA graphs from 2 ranks on, like the framework's own arm, so the
comparison is about kernels and fusion rather than host launch time (``LIB_CUDA_GRAPH=0`` turns it off).
"""
from __future__ import annotations

import json
import math
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------ tensor-parallel glue
class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty((x.shape[0] * dist.get_world_size(group),) + tuple(x.shape[1:]), dtype=x.dtype,
                          device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        n = dist.get_world_size(ctx.group)
        out = torch.empty((dy.shape[0] // n,) + tuple(dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        dist.reduce_scatter_tensor(out, dy.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        out = torch.empty((dy.shape[0] * dist.get_world_size(ctx.group),) + tuple(dy.shape[1:]), dtype=dy.dtype,
                          device=dy.device)
        dist.all_gather_into_tensor(out, dy.contiguous(), group=ctx.group)
        return out, None


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross entropy over logits sharded on the vocabulary (Megatron formulation, torch ops + all_reduce)."""

    @staticmethod
    def forward(ctx, logits, labels, start, group):
        lf = logits.float()
        m = lf.amax(-1)
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(lf - m[:, None])
        s = e.sum(-1)
        dist.all_reduce(s, group=group)
        loc = labels.long() - start
        inr = (loc >= 0) & (loc < logits.shape[-1])
        tgt = torch.where(inr, lf.gather(1, loc.clamp(0, logits.shape[-1] - 1)[:, None])[:, 0], torch.zeros_like(m))
        dist.all_reduce(tgt, group=group)
        p = e / s[:, None]
        ctx.save_for_backward(p, loc, inr)
        return (torch.log(s) + m - tgt).mean()

    @staticmethod
    def backward(ctx, dloss):
        p, loc, inr = ctx.saved_tensors
        # softmax - onehot, without data-dependent shapes (the micro-batch is captured into a CUDA graph)
        p = p.scatter_add(1, loc.clamp(0, p.shape[1] - 1)[:, None], -inr.to(p.dtype)[:, None])
        return (p * (dloss / p.shape[0])).to(torch.bfloat16), None, None, None


def _rope_tables(seq, d, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


def _rope(x, cos, sin):
    # x [B, S, H, D], rotate-half
    d = x.shape[-1]
    a, b = x[..., : d // 2].float(), x[..., d // 2:].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)


class _LlamaLayer(torch.nn.Module):
    def __init__(self, h, heads, ffn, mp, layers, dev):
        super().__init__()
        d = h // heads
        self.heads, self.d = heads // mp, d
        std = 0.02
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.attention_norm = torch.nn.Parameter(torch.ones(h, **bf))
        self.ffn_norm = torch.nn.Parameter(torch.ones(h, **bf))
        self.wqkv = torch.nn.Parameter(torch.randn(3 * h // mp, h, **bf) * std)
        self.wo = torch.nn.Parameter(torch.randn(h, h // mp, **bf) * (std / math.sqrt(2 * layers)))
        self.w_gate_up = torch.nn.Parameter(torch.randn(2 * ffn // mp, h, **bf) * std)
        self.w_down = torch.nn.Parameter(torch.randn(h, ffn // mp, **bf) * (std / math.sqrt(2 * layers)))

    def forward(self, x, cos, sin, batch, seq, group):
        h = F.rms_norm(x, (x.shape[-1],), self.attention_norm, 1e-5)
        if group is not None:
            h = _AllGatherRows.apply(h, group)
        qkv = F.linear(h, self.wqkv).view(batch, seq, 3, self.heads, self.d)
        q, k = _rope(qkv[:, :, 0], cos, sin), _rope(qkv[:, :, 1], cos, sin)
        v = qkv[:, :, 2]
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        o = F.linear(o.transpose(1, 2).reshape(batch * seq, self.heads * self.d), self.wo)
        if group is not None:
            o = _ReduceScatterRows.apply(o, group)
        x = x + o
        h = F.rms_norm(x, (x.shape[-1],), self.ffn_norm, 1e-5)
        if group is not None:
            h = _AllGatherRows.apply(h, group)
        gu = F.linear(h, self.w_gate_up)
        f = gu.shape[-1] // 2
        y = F.linear(F.silu(gu[:, :f]) * gu[:, f:], self.w_down)
        if group is not None:
            y = _ReduceScatterRows.apply(y, group)
        return x + y


class _Llama(torch.nn.Module):
    def __init__(self, layers, h, heads, ffn, vocab, mp, rank, dev):
        super().__init__()
        self.mp, self.rank, self.vocab_local = mp, rank, vocab // mp
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.tok_embeddings = torch.nn.Parameter(torch.randn(vocab // mp, h, **bf) * 0.02)
        self.layers = torch.nn.ModuleList([_LlamaLayer(h, heads, ffn, mp, layers, dev) for _ in range(layers)])
        self.norm_out = torch.nn.Parameter(torch.ones(h, **bf))
        self.lm_head = torch.nn.Parameter(torch.randn(vocab // mp, h, **bf) * 0.02)
        self.d = h // heads

    def forward(self, tokens, group):
        inp, labels = tokens[:, :-1], tokens[:, 1:]
        batch, seq = inp.shape
        cos, sin = _rope_tables(seq, self.d, 10000.0, tokens.device)
        ids = inp.reshape(-1).long()
        if group is None:
            x = F.embedding(ids, self.tok_embeddings)
        else:
            loc = ids - self.rank * self.vocab_local
            ok = (loc >= 0) & (loc < self.vocab_local)
            x = F.embedding(loc.clamp(0, self.vocab_local - 1), self.tok_embeddings) * ok[:, None].to(torch.bfloat16)
            x = _ReduceScatterRows.apply(x, group)
        for layer in self.layers:
            x = layer(x, cos, sin, batch, seq, group)
        h = F.rms_norm(x, (x.shape[-1],), self.norm_out, 1e-5)
        if group is None:
            return F.cross_entropy(F.linear(h, self.lm_head).float(), labels.reshape(-1).long())
        logits = F.linear(_AllGatherRows.apply(h, group), self.lm_head)
        return _VocabParallelCE.apply(logits, labels.reshape(-1), self.rank * self.vocab_local, group)


class _MasterAdamW:
    """bf16 parameters, fp32 master copy + moments updated by ``torch.optim.AdamW(fused=True)``, gradient clipping
    by global norm (the norm of model-parallel shards is summed over the group).  The update runs group by group
    (one group per decoder layer) so that the fp32 copy of the gradients is never resident as a whole."""

    def __init__(self, groups, lr, group, sharded):
        self.groups = [list(g) for g in groups]
        self.sharded = sharded                      # {id(param): bool}
        self.masters, self.opts = [], []
        for g in self.groups:
            m = [p.detach().float().clone().requires_grad_(True) for p in g]
            self.masters.append(m)
            self.opts.append(torch.optim.AdamW(m, lr=lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True))
        self.group = group

    def step(self, replicated_grads):
        dev = self.groups[0][0].device
        if self.group is not None and replicated_grads:
            for g in replicated_grads:
                dist.all_reduce(g, group=self.group)
        sq_sh = torch.zeros((), device=dev)
        sq_rep = torch.zeros((), device=dev)
        for grp in self.groups:
            for p in grp:
                n2 = torch.linalg.vector_norm(p.grad, dtype=torch.float32).pow(2)
                if self.sharded[id(p)]:
                    sq_sh += n2
                else:
                    sq_rep += n2
        if self.group is not None:
            dist.all_reduce(sq_sh, group=self.group)
        scale = torch.clamp(1.0 / ((sq_sh + sq_rep).sqrt() + 1e-6), max=1.0)
        for grp, masters, opt in zip(self.groups, self.masters, self.opts):
            for m, p in zip(masters, grp):
                m.grad = p.grad.float() * scale
            opt.step()
            with torch.no_grad():
                torch._foreach_copy_(grp, masters)
            for m, p in zip(masters, grp):
                m.grad = None
                p.grad.zero_()


class _GraphedMicroBatch:
    """Forward + backward of one micro-batch; after two eager calls it is captured into a CUDA graph and replayed
    (gradients accumulate in place into ``.grad``)."""

    def __init__(self, fn, enabled):
        self.fn, self.enabled, self.calls, self.graph = fn, enabled, 0, None

    def __call__(self, tokens):
        if not self.enabled:
            return self.fn(tokens)
        self.calls += 1
        if self.graph is None:
            if self.calls <= 2:
                return self.fn(tokens)
            self.static_in = tokens.clone()
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.static_out = self.fn(self.static_in)
        self.static_in.copy_(tokens)
        self.graph.replay()
        return self.static_out


def _env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def _barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _timed(step, host_batches, to_device, steps, warmup, world, sampler):
    dev_batch = to_device(host_batches(0))
    for _ in range(warmup):
        step(dev_batch)
    _barrier(world)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _barrier(world)
    e0.record()
    for _ in range(steps):
        step(dev_batch)
    e1.record()
    _barrier(world)
    dev_ms = e0.elapsed_time(e1)
    batches = [host_batches(i + 1) for i in range(steps)]
    _barrier(world)
    t0 = time.perf_counter()
    e0.record()
    last = None
    for b in batches:
        last = float(step(to_device(b)).float().cpu())
    e1.record()
    _barrier(world)
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1000)
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
    return dev_ms, e2e_ms, clocks, last, batches[0]


def run_llama(args, sampler_cls):
    world, rank, local = _env()
    dev = torch.device("cuda", local)
    torch.manual_seed(1234 + rank)
    group = dist.group.WORLD if world > 1 else None
    layers = args.layers or 32
    h, heads, ffn, vocab = 4096, 32, 11008, 32000
    net = _Llama(layers, h, heads, ffn, vocab, world, rank, dev)
    names = [n for n, _ in net.named_parameters()]
    params = [p for _, p in net.named_parameters()]
    sharded = {id(p): ("norm" not in n) for n, p in zip(names, params)}
    for p in params:
        p.grad = torch.zeros_like(p)
    groups = [list(layer.parameters()) for layer in net.layers] + [[net.tok_embeddings, net.norm_out, net.lm_head]]
    opt = _MasterAdamW(groups, 1e-4, group, sharded)
    norm_grads = [p.grad for n, p in zip(names, params) if "norm" in n]
    use_graph = os.environ.get("LIB_CUDA_GRAPH", "1") != "0" and world >= 2

    def micro(tok):
        loss = net(tok, group)
        (loss / args.global_batch).backward()
        return loss.detach()
    runner = _GraphedMicroBatch(micro, use_graph)

    def step(tokens):
        total = None
        for i in range(args.global_batch):
            li = runner(tokens[i:i + 1])
            total = li.clone() if total is None else total + li
        opt.step(norm_grads if world > 1 else None)
        return total / args.global_batch

    gen = torch.Generator().manual_seed(99)

    def host_batches(_i):
        return torch.randint(0, vocab, (args.global_batch, args.seq + 1), dtype=torch.int32, generator=gen).pin_memory()

    def to_device(b):
        return b.to(dev, non_blocking=True)

    dev_ms, e2e_ms, clocks, last, b0 = _timed(step, host_batches, to_device, args.steps, args.warmup, world,
                                              sampler_cls(local))
    if rank == 0:
        tokens_per_step = args.global_batch * args.seq
        ms_per_step = dev_ms / args.steps
        print(json.dumps({
            "impl": "library",
            "metric": "Llama-2-7B semi-auto-parallel training throughput (tokens/s, max over ranks)",
            "value": round(tokens_per_step / (ms_per_step / 1000), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 2),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": "llama2-7b" if not args.layers else "llama2-7b-truncated-%dL-INVALID" % args.layers,
                       "layers": layers, "global_batch": args.global_batch, "micro_batch": 1, "seq_len": args.seq,
                       "parallelism": "mp%d+sp" % world if world > 1 else "single",
                       "kernels": "cuBLAS F.linear, SDPA attention, torch fused AdamW, NCCL all_gather / "
                                  "reduce_scatter un-fused", "cuda_graph": use_graph,
                       "l2": "working set far larger than the 126 MB L2 (no flush needed)"},
            "clocks": clocks,
            "e2e": {"value": round(tokens_per_step / (e2e_ms / args.steps / 1000), 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": b0.numel() * b0.element_size(), "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "final_loss": last,
            "max_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}), flush=True)
    _finish(world, use_graph)
    return 0


# ------------------------------------------------------------------------------------------ ResNet-50 (DDP)
class _Bottleneck(torch.nn.Module):
    def __init__(self, cin, mid, stride):
        super().__init__()
        cout = mid * 4
        self.c1 = torch.nn.Conv2d(cin, mid, 1, bias=False)
        self.b1 = torch.nn.BatchNorm2d(mid)
        self.c2 = torch.nn.Conv2d(mid, mid, 3, stride, 1, bias=False)      # v1.5: stride on the 3x3
        self.b2 = torch.nn.BatchNorm2d(mid)
        self.c3 = torch.nn.Conv2d(mid, cout, 1, bias=False)
        self.b3 = torch.nn.BatchNorm2d(cout)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = torch.nn.Sequential(torch.nn.Conv2d(cin, cout, 1, stride, bias=False),
                                            torch.nn.BatchNorm2d(cout))

    def forward(self, x):
        idt = x if self.down is None else self.down(x)
        y = F.relu(self.b1(self.c1(x)))
        y = F.relu(self.b2(self.c2(y)))
        return F.relu(self.b3(self.c3(y)) + idt)


class _ResNet50(torch.nn.Module):
    def __init__(self, classes=1000):
        super().__init__()
        self.stem = torch.nn.Sequential(torch.nn.Conv2d(3, 64, 7, 2, 3, bias=False), torch.nn.BatchNorm2d(64),
                                        torch.nn.ReLU(), torch.nn.MaxPool2d(3, 2, 1))
        blocks, cin = [], 64
        for mid, n, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
            for i in range(n):
                blocks.append(_Bottleneck(cin, mid, stride if i == 0 else 1))
                cin = mid * 4
        self.blocks = torch.nn.Sequential(*blocks)
        self.fc = torch.nn.Linear(2048, classes)

    def forward(self, x, y):
        f = self.blocks(self.stem(x)).mean((2, 3))
        return F.cross_entropy(self.fc(f).float(), y.long(), label_smoothing=0.1)


def run_resnet(args, sampler_cls):
    world, rank, local = _env()
    dev = torch.device("cuda", local)
    torch.manual_seed(1234)
    # fp32 parameters, bf16 compute under autocast: the standard torch mixed-precision recipe (GradScaler has no
    # bf16-gradient kernel), channels_last so that cuDNN takes its tensor-core NHWC path
    net = _ResNet50().to(dev).to(memory_format=torch.channels_last)
    model = net
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(net, device_ids=[local], bucket_cap_mb=25,
                                                          gradient_as_bucket_view=True)
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4, fused=True)
    scaler = torch.amp.GradScaler("cuda", init_scale=1024.0)          # dynamic loss scaling, as the config names it
    B = args.batch_per_gpu
    gen = torch.Generator().manual_seed(7 + rank)

    def step(batch):
        x, y = batch
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(x, y)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        return loss.detach()

    def host_batches(_i):
        return (torch.randint(0, 256, (B, 224, 224, 3), dtype=torch.uint8, generator=gen).pin_memory(),
                torch.randint(0, 1000, (B,), dtype=torch.int32, generator=gen).pin_memory())

    def to_device(b):
        img, lab = b
        x = img.to(dev, non_blocking=True).permute(0, 3, 1, 2)
        return (x.to(torch.bfloat16) - 127.5) * (1.0 / 58.0), lab.to(dev, non_blocking=True)

    dev_ms, e2e_ms, clocks, last, b0 = _timed(step, host_batches, to_device, args.steps, args.warmup, world,
                                              sampler_cls(local))
    if rank == 0:
        ms_per_step = dev_ms / args.steps
        print(json.dumps({
            "impl": "library",
            "metric": "ResNet-50 v1.5 data-parallel training throughput (images/s, max over ranks)",
            "value": round(B * world / (ms_per_step / 1000), 1), "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": "resnet50-v1.5", "batch_per_gpu": B, "global_batch": B * world,
                       "parallelism": "dp%d" % world,
                       "kernels": "cuDNN convolutions / batch norm (channels_last, bf16 autocast over fp32 "
                                  "parameters), torch fused SGD, DistributedDataParallel 25 MB buckets, GradScaler "
                                  "dynamic loss scaling",
                       "l2": "activations of one step far exceed the 126 MB L2 (no flush needed)"},
            "clocks": clocks,
            "e2e": {"value": round(B * world / (e2e_ms / args.steps / 1000), 1), "unit": "images/s",
                    "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in b0), "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "final_loss": last,
            "max_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}), flush=True)
    _finish(world, False)
    return 0


def _finish(world, used_graph):
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        if used_graph:
            import sys
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)          # a live CUDA graph holds NCCL kernels of the communicator being destroyed
        dist.destroy_process_group()

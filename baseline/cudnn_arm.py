"""Library baseline for bench.py (`--impl cudnn`): the same workload with stock PyTorch operators.

Same model family, batch size, replicas per GPU, optimiser and synchronous-model-averaging arithmetic as the product arm,
but every operator is a library kernel (cuDNN convolutions with TF32 allowed, PyTorch's batch-norm kernels, cuBLAS, NCCL all-reduce), in
channels-last layout, with each replica's whole task (forward, loss, backward, momentum-SGD step) captured in a CUDA graph
and the k replicas running on k streams.  The synchronisation is reference-style: a handful of element-wise kernels over
flat parameter vectors around one `all_reduce` (what clib-multigpu/synch/sma.c does with cuBLAS level-1 calls around
ncclAllReduce).  None of this repository's kernels or engine are on this path.
"""
import copy
import os
import time

import torch
import torch.nn as nn
import torch.nn.functional as F


class _BatchNorm(nn.BatchNorm2d):
    """Batch norm through PyTorch's own kernels.  cuDNN's spatial-persistent batch-norm kernels synchronise their blocks
    with one another inside the kernel and so assume they have the GPU to themselves; with several replicas' graphs
    replaying on several streams such kernels can wait for each other for ever (this arm stalled that way with four
    replicas, always with eight).  The convolutions stay on cuDNN."""

    def forward(self, x):
        with torch.backends.cudnn.flags(enabled=False):
            return super().forward(x)


def _bn(c):
    return _BatchNorm(c, eps=1e-5, momentum=0.1)


class Basic(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.a = nn.Conv2d(cin, cout, 3, stride, 1, bias=False); self.bna = _bn(cout)
        self.b = nn.Conv2d(cout, cout, 3, 1, 1, bias=False); self.bnb = _bn(cout)
        self.short = None
        if stride != 1 or cin != cout:
            self.short = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, 0, bias=False), _bn(cout))

    def forward(self, x):
        y = F.relu(self.bna(self.a(x)))
        y = self.bnb(self.b(y))
        return F.relu(y + (x if self.short is None else self.short(x)))


class Bottleneck(nn.Module):
    def __init__(self, cin, mid, stride):
        super().__init__()
        cout = 4 * mid
        self.a = nn.Conv2d(cin, mid, 1, stride, 0, bias=False); self.bna = _bn(mid)       # stride on the first 1x1, as in models/resnet.py
        self.b = nn.Conv2d(mid, mid, 3, 1, 1, bias=False); self.bnb = _bn(mid)
        self.c = nn.Conv2d(mid, cout, 1, 1, 0, bias=False); self.bnc = _bn(cout)
        self.short = None
        if stride != 1 or cin != cout:
            self.short = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, 0, bias=False), _bn(cout))

    def forward(self, x):
        y = F.relu(self.bna(self.a(x)))
        y = F.relu(self.bnb(self.b(y)))
        y = self.bnc(self.c(y))
        return F.relu(y + (x if self.short is None else self.short(x)))


def resnet32(classes=10):
    layers, cin = [nn.Conv2d(3, 16, 3, 1, 1, bias=False), _bn(16), nn.ReLU(inplace=True)], 16
    for stage, feat in enumerate((16, 32, 64)):
        for unit in range(5):
            layers.append(Basic(cin, feat, 2 if (unit == 0 and stage > 0) else 1))
            cin = feat
    layers += [nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(64, classes)]
    return nn.Sequential(*layers)


def resnet50(classes=1000):
    layers, cin = [nn.Conv2d(3, 64, 7, 2, 3, bias=False), _bn(64), nn.ReLU(inplace=True), nn.MaxPool2d(3, 2, 0, ceil_mode=True)], 64
    for stage, (mid, units) in enumerate(((64, 3), (128, 4), (256, 6), (512, 3))):
        for unit in range(units):
            layers.append(Bottleneck(cin, mid, 2 if (unit == 0 and stage > 0) else 1))
            cin = 4 * mid
    layers += [nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(2048, classes)]
    return nn.Sequential(*layers)


def _flatten_parameters(model):
    """Re-home every parameter in one flat fp32 vector (views), so the averaging step is a few flat element-wise kernels."""
    ps = [p for p in model.parameters()]
    flat = torch.zeros(sum(p.numel() for p in ps), device=ps[0].device)
    off = 0
    for p in ps:
        n = p.numel()
        flat[off:off + n].copy_(p.data.reshape(-1))
        p.data = flat[off:off + n].view_as(p.data)
        off += n
    return flat


class Replica:
    def __init__(self, model, batch, shape, lr=0.1, momentum=0.9, wd=1e-4, graphs=True):
        self.model, self.stream = model, torch.cuda.Stream()
        self.flat = _flatten_parameters(model)
        self.prev = self.flat.clone()
        self.opt = torch.optim.SGD(model.parameters(), lr=lr, momentum=momentum, weight_decay=wd)
        self.x = torch.randn(batch, *shape, device="cuda").contiguous(memory_format=torch.channels_last)
        self.y = torch.zeros(batch, dtype=torch.long, device="cuda")
        self.loss = torch.zeros((), device="cuda")
        self.graph = None
        with torch.cuda.stream(self.stream):
            for _ in range(3):                              # warm-up outside capture (allocations, cuDNN algorithm search)
                self._task()
        torch.cuda.synchronize()
        if graphs:
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    self._task()
                self.graph = g
            except Exception:
                self.graph = None
        torch.cuda.synchronize()

    def _task(self):
        self.prev.copy_(self.flat)                          # pre-update snapshot, as the product arm keeps
        self.opt.zero_grad(set_to_none=False)
        out = self.model(self.x)
        loss = F.cross_entropy(out, self.y)
        loss.backward()
        self.opt.step()
        self.loss.copy_(loss.detach())

    def run(self):
        with torch.cuda.stream(self.stream):
            if self.graph is not None:
                self.graph.replay()
            else:
                self._task()


def run(args, cfg, json_out):
    """Stand-alone arm (`bench.py --impl cudnn`): measure, print the JSON line, leave the process group."""
    import torch.distributed as dist
    out = measure(args, cfg, getattr(args, "min_seconds", 0.0))
    if int(os.environ.get("RANK", 0)) == 0:
        print(json_out(out))
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


def measure(args, cfg, min_seconds=0.0):
    """Run the library arm in this process (joining the existing process group if there is one) and return its record.
    `min_seconds`: repeat the timed block of `args.steps` steps until that much time has been measured; the reported
    value is the median repeat."""
    import torch.distributed as dist
    torch.backends.cudnn.benchmark = True
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cuda.matmul.allow_tf32 = True
    world, rank, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=180))
    k, batch = args.replicas or cfg["replicas"], args.batch or cfg["batch"]
    build = {"resnet32": resnet32, "resnet50": resnet50}.get(args.model)
    if build is None:
        return {"impl": "cudnn", "unavailable": f"no library arm for {args.model}"}
    if k > 4:
        # eight captured graphs replaying on eight streams did not finish within 15 minutes on this pool (cause not found);
        # the arm is only run at the replica counts that were seen to complete
        return {"impl": "cudnn", "unavailable": "library arm is limited to 4 replicas per GPU"}
    torch.manual_seed(1)
    base = build(cfg["classes"]).cuda().to(memory_format=torch.channels_last).train()
    reps = [Replica(copy.deepcopy(base), batch, cfg["shape"], graphs=not args.no_graphs) for _ in range(k)]
    z = reps[0].flat.clone()
    zlast = torch.zeros_like(z)
    acc = torch.zeros_like(z)
    sync_stream = torch.cuda.Stream()
    alpha, mu = 0.1, 0.9
    pinned_x = [torch.randn(batch, *cfg["shape"]).contiguous(memory_format=torch.channels_last).pin_memory() for _ in range(max(2 * k, 8))]
    pinned_y = [torch.randint(0, cfg["classes"], (batch,)).pin_memory() for _ in range(len(pinned_x))]

    def synchronise():
        # reference-style: per-replica element-wise kernels, one all-reduce, central update with momentum
        for r in reps:
            sync_stream.wait_stream(r.stream)
        with torch.cuda.stream(sync_stream):
            acc.zero_()
            for r in reps:
                d = (r.prev - z).mul_(alpha)
                r.flat.sub_(d)
                acc.add_(d)
            if world > 1:
                dist.all_reduce(acc)
            zlast.mul_(mu).add_(acc)
            z.add_(zlast)
        for r in reps:
            r.stream.wait_stream(sync_stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def mx(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def step(e2e, i):
        losses = []
        for j, r in enumerate(reps):
            if e2e:
                s = (i * k + j) % len(pinned_x)
                with torch.cuda.stream(r.stream):
                    r.x.copy_(pinned_x[s], non_blocking=True)
                    r.y.copy_(pinned_y[s], non_blocking=True)
            r.run()
        synchronise()
        if e2e:
            for r in reps:
                r.stream.synchronize()
                losses.append(float(r.loss))
        return losses

    def timed_device():
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(sync_stream)
        for i in range(args.steps):
            step(False, i)
        for r in reps:
            sync_stream.wait_stream(r.stream)
        e1.record(sync_stream)
        e1.synchronize()
        barrier()
        return mx(e0.elapsed_time(e1))

    def timed_e2e():
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            step(True, i)
        torch.cuda.synchronize()
        return mx(time.perf_counter() - t0) * 1e3

    def repeat(fn):
        first = fn()
        n = max(1, min(50, int(-(-min_seconds * 1e3 // max(first, 1e-3))))) if min_seconds > 0 else 1
        v = sorted([first] + [fn() for _ in range(n - 1)])
        return v[len(v) // 2], v

    sampler = None
    if getattr(args, "clock_sampler", None) is not None:
        sampler = args.clock_sampler(local)
        sampler.start()
    for i in range(max(3, args.warmup)):
        step(False, i)
    dev_ms, dev_all = repeat(timed_device)
    for i in range(3):
        step(True, i)
    e2e_ms, e2e_all = repeat(timed_e2e)
    barrier()
    if sampler is not None:
        sampler.stop_flag.set()
        sampler.join(timeout=2)
    images = batch * k * world
    out = {
        "metric": f"{args.model} SMA training throughput", "value": round(images * args.steps / (dev_ms / 1e3), 1), "unit": "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(dev_ms / args.steps, 4),
        "repeats": len(dev_all), "ms_per_step_min_max": [round(dev_all[0] / args.steps, 4), round(dev_all[-1] / args.steps, 4)],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32 (cuDNN / cuBLAS), fp32 storage",
        "data": "synthetic", "impl": "cudnn",
        "config": {"model": args.model, "global_batch": images, "batch_per_replica": batch, "replicas_per_gpu": k,
                   "parallelism": f"dp{world} x {k} replicas/GPU, SMA alpha 0.1, wpc = k*G", "sync": "element-wise kernels + NCCL all-reduce",
                   "cuda_graphs": reps[0].graph is not None, "layout": "channels_last"},
        "e2e": {"value": round(images * args.steps / (e2e_ms / 1e3), 1), "unit": "images/s", "repeats": len(e2e_all),
                "h2d_bytes_per_step": k * batch * (4 * int(torch.tensor(cfg["shape"]).prod()) + 8), "d2h_bytes_per_step": 4 * k},
        "gpu_launches": 0, "note": "library kernels only: none of this repository's kernels run in this arm"}
    if sampler is not None:
        out["clocks"] = sampler.summary()
    del reps
    torch.cuda.empty_cache()
    return out

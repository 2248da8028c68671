"""Per-kernel micro-benchmark: times one native kernel with CUDA events and reports achieved bandwidth / FLOP rate
against the measured peaks of the machine (``MEASURED_PEAKS.json`` at the repository root when present).

    python -m crossbow_b200.ops.kernel_bench --op conv_fprop --impl tc --shape 64,32,32,16,16,3,3,1,1
    python -m crossbow_b200.ops.kernel_bench --op bn_fwd --rows 65536 --channels 16
    python -m crossbow_b200.ops.kernel_bench --op sync --n 25600000 --replicas 2
    python -m crossbow_b200.ops.kernel_bench --suite resnet32

Timing protocol: 3 warm-up launches, then CUDA events on the launching stream around ``--iters`` repetitions of
[overwrite a 256 MB buffer, launch], minus the same loop without the launch: every launch starts with a cold L2 (the
tensors of these small-batch layers are far smaller than the 126 MB L2) and an idle stream's launch latency is not
charged to the kernel.  The median of three such spans is reported.  ``--warm`` drops the flush and reports the
L2-resident back-to-back time, which is what a kernel sees inside a training task.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics

import torch

from . import lib as L


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    """Device time per launch = (events around `iters` x [flush, launch]) minus (events around `iters` x [flush]),
    so neither the host launch latency of an idle stream nor the flush itself is attributed to the kernel."""

    def __init__(self, flush=True):
        self.flush = torch.empty(64 << 20, device="cuda") if flush else None    # 256 MB > 126 MB L2
        self.s = torch.cuda.current_stream()

    def _span(self, body, iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record(self.s)
        for _ in range(iters):
            body()
        b.record(self.s)
        b.synchronize()
        return a.elapsed_time(b) * 1e3 / iters

    def run(self, fn, iters=20, warmup=3):
        for _ in range(warmup):
            fn()
        if self.flush is None:
            ts = [self._span(fn, iters) for _ in range(3)]
            return statistics.median(ts), min(ts)
        fl = lambda: self.flush.fill_(1.0)

        def both():
            fl()
            fn()
        base = min(self._span(fl, iters) for _ in range(3))
        ts = [self._span(both, iters) - base for _ in range(3)]
        return statistics.median(ts), min(ts)


def geom(N, H, W, Cc, K, R, S, st, pad):
    g = L.XbConvGeom()
    P, Q = (H + 2 * pad - R) // st + 1, (W + 2 * pad - S) // st + 1
    g.N, g.H, g.W, g.C, g.K, g.R, g.S, g.P, g.Q, g.sh, g.sw, g.ph, g.pw = N, H, W, Cc, K, R, S, P, Q, st, st, pad, pad
    return g, P, Q


def bench_conv(lib, timer, op, impl, shape, iters, flags=0):
    N, H, W, Cc, K, R, S, st, pad = shape
    g, P, Q = geom(*shape)
    dev = "cuda"
    x = torch.randn(N, H, W, Cc, device=dev)
    w = torch.randn(K, R, S, Cc, device=dev) * 0.05
    wt = w.permute(3, 1, 2, 0).contiguous()
    y = torch.empty(N, P, Q, K, device=dev)
    dy = torch.randn(N, P, Q, K, device=dev)
    dx = torch.empty_like(x)
    dw = torch.zeros_like(w)
    stats = torch.zeros(2 * K, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    s = torch.cuda.current_stream().cuda_stream
    gp = C.byref(g)
    if op == "conv_fprop":
        if impl == "tc":
            fn = lambda: lib.xb_conv_fprop_tc(x.data_ptr(), w.data_ptr(), 0, y.data_ptr(), stats.data_ptr(), gp, flags, status.data_ptr(), s)
        else:
            fn = lambda: lib.xb_conv_fprop_simt(x.data_ptr(), w.data_ptr(), 0, y.data_ptr(), stats.data_ptr(), gp, flags, s)
        bytes_ = 4 * (x.numel() + w.numel() + y.numel())
    elif op == "conv_dgrad":
        if impl == "tc":
            fn = lambda: lib.xb_conv_dgrad_tc(dy.data_ptr(), wt.data_ptr(), dx.data_ptr(), gp, 0, status.data_ptr(), s, None)
        else:
            fn = lambda: lib.xb_conv_dgrad_simt(dy.data_ptr(), wt.data_ptr(), dx.data_ptr(), gp, 0, s)
        bytes_ = 4 * (dy.numel() + w.numel() + dx.numel())
    else:
        if impl == "tc":
            fn = lambda: lib.xb_conv_wgrad_tc(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), gp, status.data_ptr(), s)
        else:
            fn = lambda: lib.xb_conv_wgrad_simt(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), gp, s)
        bytes_ = 4 * (dy.numel() + x.numel() + 2 * dw.numel())
    e = fn()
    L.check(e, op)
    med, best = timer.run(fn, iters)
    torch.cuda.synchronize()
    if int(status[0]) != 0:
        raise RuntimeError("kernel reported a bounded-wait expiry")
    flops = 2.0 * N * P * Q * K * R * S * Cc
    return dict(op=op, impl=impl, shape=list(shape), us=round(med, 2), best_us=round(best, 2), bytes=bytes_, flops=flops)


def bench_bn(lib, timer, op, M, Cc, iters):
    dev = "cuda"
    x, y, dy, dx = (torch.randn(M, Cc, device=dev) for _ in range(4))
    sums, dsums = torch.zeros(2 * Cc, device=dev), torch.zeros(2 * Cc, device=dev)
    gamma, beta, rm, rv, sm, si = torch.ones(Cc, device=dev), torch.zeros(Cc, device=dev), torch.zeros(Cc, device=dev), \
        torch.ones(Cc, device=dev), torch.zeros(Cc, device=dev), torch.ones(Cc, device=dev)
    dg, db = torch.zeros(Cc, device=dev), torch.zeros(Cc, device=dev)
    tp = torch.zeros(16, dtype=torch.int32, device=dev)
    s = torch.cuda.current_stream().cuda_stream
    lib.xb_bn_stats(x.data_ptr(), sums.data_ptr(), M, Cc, s)
    if op == "bn_fwd":
        fn = lambda: lib.xb_bn_forward(x.data_ptr(), 0, y.data_ptr(), sums.data_ptr(), gamma.data_ptr(), beta.data_ptr(), rm.data_ptr(),
                                       rv.data_ptr(), sm.data_ptr(), si.data_ptr(), tp.data_ptr(), M, Cc, 1e-5, 1, 1, 0, 0.1, s)
        bytes_ = 8 * M * Cc
    elif op == "bn_stats":
        fn = lambda: lib.xb_bn_stats(x.data_ptr(), sums.data_ptr(), M, Cc, s)
        bytes_ = 4 * M * Cc
    elif op in ("bn_bwd_res", "bn_bwd_res_mask"):
        # layer with ReLU and a residual input: the mask comes from the output y, or from the packed sign bytes
        dres = torch.empty(M, Cc, device=dev)
        mask = torch.randint(0, 16, (M * Cc // 4,), dtype=torch.uint8, device=dev)
        packed = op.endswith("mask")
        ysrc, relu = (mask, 3) if packed else (y, 1)
        fn = lambda: lib.xb_bn_backward(dy.data_ptr(), x.data_ptr(), ysrc.data_ptr(), sm.data_ptr(), si.data_ptr(), gamma.data_ptr(), dsums.data_ptr(),
                                        dx.data_ptr(), dres.data_ptr(), dg.data_ptr(), db.data_ptr(), M, Cc, relu, 0, 0, s)
        # reduce reads dy, x, mask source; apply reads the same and writes dx and dres
        bytes_ = 4 * M * Cc * 6 + 2 * (M * Cc // 4 if packed else 4 * M * Cc)
    else:
        fn = lambda: lib.xb_bn_backward(dy.data_ptr(), x.data_ptr(), y.data_ptr(), sm.data_ptr(), si.data_ptr(), gamma.data_ptr(), dsums.data_ptr(),
                                        dx.data_ptr(), 0, dg.data_ptr(), db.data_ptr(), M, Cc, 1, 0, 0, s)
        bytes_ = 4 * M * Cc * 7     # reduce reads dy,x,y; apply reads dy,x,y and writes dx
    L.check(fn(), op)
    med, best = timer.run(fn, iters)
    return dict(op=op, rows=M, channels=Cc, us=round(med, 2), best_us=round(best, 2), bytes=bytes_, flops=0)


def bench_image(lib, timer, n, W, H, S, iters):
    """Crop / mirror / bilinear resize / scaling of `n` decoded W x H images into S x S examples (csrc/kernels/image.cu)."""
    import numpy as np
    g = np.random.default_rng(0)
    stride = (W * H * 3 + 15) // 16 * 16
    rgb = torch.randint(0, 256, (n * stride,), dtype=torch.uint8, device="cuda")
    desc = np.zeros((n, lib.xb_image_desc_size() // 4), dtype=np.int32)
    for i in range(n):
        cw, ch = int(g.integers(W // 3, W + 1)), int(g.integers(H // 3, H + 1))
        desc[i].view(np.int64)[0] = i * stride
        desc[i, 2:9] = (W, H, int(g.integers(0, W - cw + 1)), int(g.integers(0, H - ch + 1)), cw, ch, int(g.integers(0, 2)))
    d = torch.from_numpy(desc).cuda()
    out = torch.empty(n, 3, S, S, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    fn = lambda: lib.xb_image_crop_resize(rgb.data_ptr(), d.data_ptr(), n, S, out.data_ptr(), s)
    L.check(fn(), "image")
    med, best = timer.run(fn, iters)
    # every output value reads (up to) four source bytes that are mostly shared with its neighbours: the output dominates
    return dict(op="image_crop_resize", images=n, source=[W, H], size=S, us=round(med, 2), best_us=round(best, 2), bytes=12 * n * S * S + int(desc[:, 6].astype(np.int64) @ desc[:, 7].astype(np.int64)) * 3, flops=0)


def bench_sync(lib, timer, n, k, iters):
    from ..parallel.sync import ALGO_SMA, FusedSynchroniser
    dev = "cuda"
    n = (n + 3) // 4 * 4
    ws = [torch.randn(n, device=dev) * 0.01 for _ in range(k)]
    ps = [torch.randn(n, device=dev) * 0.01 for _ in range(k)]
    z, zl = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    fs = FusedSynchroniser(n)
    s = torch.cuda.current_stream().cuda_stream
    fn = lambda: fs.synchronise(s, ALGO_SMA, ws, ps, z, zl, alpha=0.1, mu=0.9)
    med, best = timer.run(fn, iters)
    fs.check()
    bytes_ = 4 * n * (3 * k + 4)    # per replica: read prev, read+write w; z and z_last read+write
    return dict(op="sync_sma_1gpu", n=n, replicas=k, us=round(med, 2), best_us=round(best, 2), bytes=bytes_, flops=0)


def bench_optimiser(lib, timer, n, iters):
    dev = "cuda"
    n = (n + 3) // 4 * 4
    w, g, last, prev = (torch.randn(n, device=dev) * 0.01 for _ in range(4))
    tp = L.XbTaskParams()
    tp.lr, tp.momentum, tp.weight_decay, tp.clip = 0.1, 0.9, 1e-4, -1.0
    tpd = torch.frombuffer(bytearray(bytes(tp)), dtype=torch.uint8).to(dev)
    s = torch.cuda.current_stream().cuda_stream
    fn = lambda: lib.xb_fused_optimiser(w.data_ptr(), g.data_ptr(), last.data_ptr(), prev.data_ptr(), 0, 0, 0, tpd.data_ptr(), n, 0, s)
    L.check(fn(), "optimiser")
    med, best = timer.run(fn, iters)
    return dict(op="fused_optimiser", n=n, us=round(med, 2), best_us=round(best, 2), bytes=4 * n * 7, flops=0)


def bench_pointwise(lib, timer, op, iters):
    """Element-wise / pooling / loss kernels on the shapes they have in ResNet-50 (batch 32) and VGG-16 (batch 128)."""
    dev = "cuda"
    s = torch.cuda.current_stream().cuda_stream
    tp = L.XbTaskParams()
    tp.training, tp.task_id, tp.seed_lo = 1, 3, 17
    tpd = torch.frombuffer(bytearray(bytes(tp)), dtype=torch.uint8).to(dev)
    if op in ("relu_fwd", "relu_bwd", "dropout"):
        n = 32 * 56 * 56 * 256 if op != "dropout" else 128 * 32 * 32 * 64
        x, y, dy, dx = (torch.randn(n, device=dev) for _ in range(4))
        if op == "relu_fwd":
            fn, bytes_ = (lambda: lib.xb_act_forward(x.data_ptr(), y.data_ptr(), n, 0, 0.0, 0.0, s)), 8 * n
        elif op == "relu_bwd":
            fn, bytes_ = (lambda: lib.xb_act_backward(dy.data_ptr(), x.data_ptr(), y.data_ptr(), dx.data_ptr(), n, 0, 0.0, 0.0, 0, s)), 12 * n
        else:
            fn, bytes_ = (lambda: lib.xb_dropout(x.data_ptr(), y.data_ptr(), n, 0.3, 5, tpd.data_ptr(), 0, s)), 8 * n
        shape = [n]
    elif op in ("maxpool_fwd", "maxpool_bwd", "avgpool_fwd"):
        if op == "avgpool_fwd":
            N, H, W, Cc, R, st = 32, 7, 7, 2048, 7, 1
        else:
            N, H, W, Cc, R, st = 32, 112, 112, 64, 3, 2
        P = -(-(H - R) // st) + 1                      # ceil mode, no padding (the reference's ResNet-50 pooling)
        geo = (C.c_int * 12)(N, H, W, Cc, P, P, R, R, st, st, 0, 0)
        x, dx = torch.randn(N * H * W * Cc, device=dev), torch.empty(N * H * W * Cc, device=dev)
        y, dy = torch.empty(N * P * P * Cc, device=dev), torch.randn(N * P * P * Cc, device=dev)
        if op == "maxpool_bwd":
            fn, bytes_ = (lambda: lib.xb_pool_backward(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), geo, 0, 0, s)), 4 * (dy.numel() + 3 * x.numel())
        else:
            fn, bytes_ = (lambda: lib.xb_pool_forward(x.data_ptr(), y.data_ptr(), geo, int(op == "avgpool_fwd"), s)), 4 * (x.numel() + y.numel())
        shape = [N, H, W, Cc, R, st]
    elif op == "softmax_xent":
        rows, classes = 32, 1000
        logits, probs, dl = torch.randn(rows, classes, device=dev), torch.empty(rows, classes, device=dev), torch.empty(rows, classes, device=dev)
        labels, res = torch.randint(0, classes, (rows,), dtype=torch.int32, device=dev), torch.zeros(2, device=dev)
        fn = lambda: lib.xb_softmax_xent(logits.data_ptr(), labels.data_ptr(), probs.data_ptr(), dl.data_ptr(), res.data_ptr(), rows, classes, -1, 0, 0, 1, s)
        bytes_, shape = 12 * rows * classes, [rows, classes]
    else:
        raise SystemExit(f"unknown op {op}")
    L.check(fn(), op)
    med, best = timer.run(fn, iters)
    return dict(op=op, shape=shape, us=round(med, 2), best_us=round(best, 2), bytes=bytes_, flops=0)


POINTWISE = ("relu_fwd", "relu_bwd", "dropout", "maxpool_fwd", "maxpool_bwd", "avgpool_fwd", "softmax_xent")
# inner-product layers as the GEMM sees them (rows = batch): VGG-16 512 -> 512 at batch 128, ResNet-50 2048 -> 1000 at batch 32
FC_SHAPES = [(128, 1, 1, 512, 512, 1, 1, 1, 0), (32, 1, 1, 2048, 1000, 1, 1, 1, 0)]


def report(r):
    bw, tf, how = peaks()
    us = r["us"]
    r["gbs"] = round(r["bytes"] / us / 1e3, 1)
    r["frac_hbm"] = round(r["gbs"] / bw, 3)
    if r.get("flops"):
        r["tflops"] = round(r["flops"] / us / 1e6, 2)
        r["frac_bf16_gemm_peak"] = round(r["tflops"] / tf, 4)
    r["peaks"] = how
    print(json.dumps(r))


RESNET32 = [(64, 32, 32, 16, 16, 3, 3, 1, 1), (64, 32, 32, 16, 32, 3, 3, 2, 1), (64, 16, 16, 32, 32, 3, 3, 1, 1),
            (64, 16, 16, 32, 64, 3, 3, 2, 1), (64, 8, 8, 64, 64, 3, 3, 1, 1)]
RESNET50 = [(32, 56, 56, 64, 64, 1, 1, 1, 0), (32, 56, 56, 64, 64, 3, 3, 1, 1), (32, 56, 56, 64, 256, 1, 1, 1, 0),
            (32, 28, 28, 128, 128, 3, 3, 1, 1), (32, 14, 14, 256, 256, 3, 3, 1, 1), (32, 14, 14, 1024, 256, 1, 1, 1, 0),
            (32, 7, 7, 512, 512, 3, 3, 1, 1), (32, 7, 7, 512, 2048, 1, 1, 1, 0)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="conv_fprop")
    ap.add_argument("--impl", default="tc")
    ap.add_argument("--shape", default="64,32,32,16,16,3,3,1,1", help="N,H,W,C,K,R,S,stride,pad")
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--channels", type=int, default=16)
    ap.add_argument("--n", type=int, default=464154)
    ap.add_argument("--replicas", type=int, default=2)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warm", action="store_true", help="do not flush L2 between launches")
    ap.add_argument("--stats", action="store_true", help="convolution epilogue also produces batch-norm sums")
    ap.add_argument("--opt-blocks", type=int, default=0, help="tuning: blocks of the fused optimiser kernel")
    ap.add_argument("--no-split-k", action="store_true", help="A/B: inner products keep their whole reduction in one CTA")
    ap.add_argument("--suite", default=None, choices=[None, "resnet32", "resnet50", "pointwise"])
    a = ap.parse_args()
    lib = L.init_device()
    lib.xb_tc_set_slab(3)
    if a.opt_blocks:
        lib.xb_optimiser_set_blocks(a.opt_blocks)
    if a.no_split_k:
        lib.xb_gemm_set_split_k(0)
    timer = Timer(flush=not a.warm)
    if a.suite == "pointwise":
        for op in POINTWISE:
            report(bench_pointwise(lib, timer, op, a.iters))
        for sh in FC_SHAPES:
            for op in ("conv_fprop", "conv_dgrad", "conv_wgrad"):
                g, _, _ = geom(*sh)
                impl = "tc" if lib.xb_tc_supported(C.byref(g), {"conv_fprop": 0, "conv_dgrad": 1, "conv_wgrad": 2}[op]) else "simt"
                report(bench_conv(lib, timer, op, impl, sh, a.iters))
        return
    if a.suite:
        shapes = RESNET32 if a.suite == "resnet32" else RESNET50
        for sh in shapes:
            for op in ("conv_fprop", "conv_dgrad", "conv_wgrad"):
                for impl in ("simt", "tc"):
                    g, _, _ = geom(*sh)
                    which = {"conv_fprop": 0, "conv_dgrad": 1, "conv_wgrad": 2}[op]
                    if impl == "tc" and not lib.xb_tc_supported(C.byref(g), which):
                        continue
                    report(bench_conv(lib, timer, op, impl, sh, a.iters, 4 if (a.stats and op == "conv_fprop") else 0))
        for M, Cc in ((65536, 16), (16384, 32), (4096, 64)) if a.suite == "resnet32" else ((100352, 64), (100352, 256), (6272, 1024)):
            for op in ("bn_fwd", "bn_bwd"):
                report(bench_bn(lib, timer, op, M, Cc, a.iters))
        n = 464154 if a.suite == "resnet32" else 25557032
        report(bench_optimiser(lib, timer, n, a.iters))
        for k in (1, 2, 4):
            report(bench_sync(lib, timer, n, k, a.iters))
        return
    if a.op.startswith("conv"):
        report(bench_conv(lib, timer, a.op, a.impl, tuple(int(v) for v in a.shape.split(",")), a.iters, 4 if a.stats else 0))
    elif a.op.startswith("bn"):
        report(bench_bn(lib, timer, a.op, a.rows, a.channels, a.iters))
    elif a.op == "image":
        report(bench_image(lib, timer, a.rows, 500, 375, 224, a.iters))
    elif a.op == "sync":
        report(bench_sync(lib, timer, a.n, a.replicas, a.iters))
    elif a.op == "optimiser":
        report(bench_optimiser(lib, timer, a.n, a.iters))
    elif a.op in POINTWISE:
        report(bench_pointwise(lib, timer, a.op, a.iters))
    else:
        raise SystemExit(f"unknown op {a.op}")


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Forward + backward timing of the convnet-benchmarks models (AlexNet v2, OverFeat, VGG-A, and an Inception-style net),
the counterpart of the reference's convnet/benchmarks/App.java:86-107.

    python examples/convnet_benchmarks.py --model alexnet --batch 128 --iters 10
    python examples/convnet_benchmarks.py --benchmark oxfordnet --forward-only true      (the reference's flag names)
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="alexnet", choices=["alexnet", "overfeat", "vgg-a", "googlenet", "mini-inception", "inception-v3"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--benchmark", default=None, help="the reference's name of --model: alexnet, overfeat, oxfordnet / vgga, googlenet")
    ap.add_argument("--forward-only", default="false", help="true: time the forward pass alone (the test graph)")
    a = ap.parse_args()
    if a.benchmark:
        a.model = {"oxfordnet": "vgg-a", "vgga": "vgg-a"}.get(a.benchmark, a.benchmark)
    forward_only = str(a.forward_only).lower() in ("true", "1", "yes")
    import torch
    from crossbow_b200 import Model, Phase, Shape, SolverConf, UpdateModel
    from crossbow_b200.engine import GpuEngine
    from crossbow_b200.models import build
    solver = SolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.01)
    spec = build(a.model, solver_conf=solver)
    m = Model()
    nid = spec.train.init(Shape([a.batch] + spec.input_shape), Shape([a.batch]), m)
    m.finalise()
    if forward_only:
        spec.test.init(Shape([a.batch] + spec.input_shape), Shape([a.batch]), m, nid)
    eng = GpuEngine(spec.train, spec.test if forward_only else None, m, m.initial_values(1), a.batch, spec.input_shape, solver, UpdateModel.DEFAULT,
                    replicas=1, wpc=1)
    phase = Phase.CHECK if forward_only else Phase.TRAIN
    x = torch.randn(a.batch, *spec.input_shape).pin_memory()
    y = torch.randint(0, spec.classes, (a.batch,), dtype=torch.int32).pin_memory()
    for _ in range(3):
        eng.submit(0, x, y, 0, phase)
        eng.wait(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for t in range(a.iters):
        eng.submit(0, x, y, t, phase)
        eng.wait(0)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    print(json.dumps({"model": a.model, "batch": a.batch, ("ms_per_iteration_fwd" if forward_only else "ms_per_iteration_fwd_bwd_update"): round(ms, 3), "images_per_s": round(a.batch / ms * 1e3, 1)}))
    eng.destroy()


if __name__ == "__main__":
    main()

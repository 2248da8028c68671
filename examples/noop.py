#!/usr/bin/env python
"""The reference's no-op applications (NoopApp.java:20-140, NoopStatelessApp.java): a chain of `--chain` operators that copy
their input, driven through the whole runtime, to see what the scheduler, the data path and the result path cost per
task when the model does (nearly) nothing.

    python examples/noop.py --chain 10 --N 2000 --training-unit tasks --gpu true --number-of-gpu-models 2
    python examples/noop.py --chain 2 --stateless true --gpu false --cpu true        (operators without a model variable)

`--dataset-alias cifar-10|imagenet` picks the input shape (3x32x32 or 3x224x224); the data is synthetic unless
`--metadata <file>` names a binary data set.
"""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from crossbow_b200 import (Dataflow, DataflowNode, ModelConf, Noop, NoopConf, NoopStateless, Operator, Phase, SubGraph, SystemConf,  # noqa: E402
                           TrainingUnit)
from crossbow_b200.cli import CommandLine, Option, Options  # noqa: E402
from crossbow_b200.context import ExecutionContext  # noqa: E402
from crossbow_b200.data import SyntheticDataset  # noqa: E402


def main(argv=None):
    opts = Options("noop.py")
    opts.add(Option("--N", int, 2)).add(Option("--training-unit", str, "tasks")).add(Option("--chain", int, 10))
    opts.add(Option("--dataset-alias", str, "cifar-10")).add(Option("--stateless", str, "false")).add(Option("--metadata", str, None))
    # the reference's defaults for this application: one replica, no synchronisation within a run, a quiet display
    SystemConf.getInstance().setDisplayInterval(10000)
    ModelConf.getInstance().setBatchSize(64).setWpc(10000000).setSlack(0)
    ModelConf.getInstance().getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.01).setMomentum(0)
    CommandLine(opts).parse(argv)
    sysc, mc = SystemConf.getInstance(), ModelConf.getInstance()
    alias = opts.get("--dataset-alias").get().lower()
    if alias not in ("cifar-10", "imagenet"):
        raise SystemExit(f"error: invalid dataset alias: {alias}")
    shape = [3, 32, 32] if alias == "cifar-10" else [3, 224, 224]
    if opts.get("--metadata").get():
        from crossbow_b200.data.native import BasicDataset
        train = BasicDataset(opts.get("--metadata").get(), window=sysc.mapped_partitions_window, register_with_cuda=sysc.gpu)
    else:
        train = SyntheticDataset(shape, 10, mc.batch_size, batches=32, seed=sysc.random_seed)
    mc.setDataset(Phase.TRAIN, train).setDataset(Phase.CHECK, None)
    stateless = str(opts.get("--stateless").get()).lower() in ("true", "1", "yes")
    make = (lambda: NoopStateless(NoopConf().setAxis(3))) if stateless else (lambda: Noop(NoopConf().setAxis(3)))
    head = node = DataflowNode(Operator("Noop-1", make()))
    for i in range(1, max(1, opts.get("--chain").get())):
        node = node.connectTo(DataflowNode(Operator(f"Noop-{i + 1}", make())))
    ctx = ExecutionContext([Dataflow(SubGraph(head)).setPhase(Phase.TRAIN), None], quiet=True)
    ctx.init()
    n, unit = opts.get("--N").get(), TrainingUnit.from_string(opts.get("--training-unit").get())
    ctx.train(min(8, ctx._tasks_of(n, unit)), TrainingUnit.TASKS)                  # warm-up (graphs, buffers)
    t0 = time.perf_counter()
    done = ctx.train(n, unit)
    dt = time.perf_counter() - t0
    print(json.dumps({"chain": opts.get("--chain").get(), "stateless": stateless, "tasks": done, "seconds": round(dt, 4),
                      "tasks_per_s": round(done / dt, 1), "us_per_task": round(dt / max(done, 1) * 1e6, 1), "batch": mc.batch_size,
                      "input": shape, "replicas": sysc.number_of_gpu_models if sysc.gpu else sysc.number_of_cpu_models}))
    ctx.destroy()


if __name__ == "__main__":
    main()

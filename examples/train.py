#!/usr/bin/env python
"""Train any model of the zoo from the command line with the reference's flags, e.g. (scripts/benchmarks/resnet-32.sh):

    python examples/train.py --model resnet32 --gpu true --number-of-gpu-models 2 --batch-size 64 --wpc 2 \
        --update-model SMA --alpha 0.1 --learning-rate 0.1 --momentum 0.9 --weight-decay 0.0001 \
        --learning-rate-decay-policy multistep --step-values 80,120 --learning-rate-step-unit epochs --gamma 0.1 \
        --N 2 --training-unit epochs

Multi-GPU: ``python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train.py ...``.
Data: ``--metadata <file>`` of a binary data set written by ``DatasetWriter``; without it a synthetic data set of the
model's input shape is generated.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from crossbow_b200 import Dataflow, ModelConf, Phase, SystemConf, TrainingUnit  # noqa: E402
from crossbow_b200.cli import CommandLine, Option, Options  # noqa: E402
from crossbow_b200.context import ExecutionContext  # noqa: E402
from crossbow_b200.data import SyntheticDataset  # noqa: E402
from crossbow_b200.models import build  # noqa: E402


def main(argv=None):
    opts = Options("train.py")
    opts.add(Option("--model", str, "resnet32")).add(Option("--N", int, 1)).add(Option("--training-unit", str, "epochs"))
    opts.add(Option("--metadata", str, None)).add(Option("--test-metadata", str, None)).add(Option("--synthetic-batches", int, 64))
    opts.add(Option("--target-loss", float, 0.0))
    CommandLine(opts).parse(argv)
    sysc, mc = SystemConf.getInstance(), ModelConf.getInstance()
    spec = build(opts.get("--model").get(), solver_conf=mc.getSolverConf())
    if int(os.environ.get("WORLD_SIZE", 1)) > 1:      # one process per GPU (nccl) or per CPU device group (gloo)
        from crossbow_b200.parallel.peer import init_process_group
        init_process_group()
    if opts.get("--metadata").get():
        from crossbow_b200.data.native import BasicDataset
        train = BasicDataset(opts.get("--metadata").get(), window=sysc.mapped_partitions_window, register_with_cuda=sysc.gpu)
        test = BasicDataset(opts.get("--test-metadata").get(), window=sysc.mapped_partitions_window, register_with_cuda=sysc.gpu) \
            if opts.get("--test-metadata").get() else None
    else:
        train = SyntheticDataset(spec.input_shape, spec.classes, mc.batch_size, batches=opts.get("--synthetic-batches").get(), seed=sysc.random_seed)
        test = SyntheticDataset(spec.input_shape, spec.classes, mc.batch_size, batches=8, seed=sysc.random_seed + 1)
    mc.setDataset(Phase.TRAIN, train).setDataset(Phase.CHECK, test)
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), Dataflow(spec.test).setPhase(Phase.CHECK) if test is not None else None])
    ctx.init()
    print(sysc.dump())
    print(mc.dump())
    print(ctx.model.dump().splitlines()[0])
    n, unit = opts.get("--N").get(), TrainingUnit.from_string(opts.get("--training-unit").get())
    if opts.get("--target-loss").get() > 0:
        ctx.trainUntilCondition(opts.get("--target-loss").get(), ctx._tasks_of(n, unit))
    elif test is not None:
        ctx.trainAndTest(n, unit)
    else:
        ctx.train(n, unit)
    if sysc.checkpoint_directory:
        print("checkpoint:", ctx.checkpoint())
    ctx.destroy()


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Train any model of the zoo from the command line with the reference's flags, e.g. (scripts/benchmarks/resnet-32.sh):

    python examples/train.py --model resnet32 --gpu true --number-of-gpu-models 2 --batch-size 64 --wpc 2 \
        --update-model SMA --alpha 0.1 --learning-rate 0.1 --momentum 0.9 --weight-decay 0.0001 \
        --learning-rate-decay-policy multistep --step-values 80,120 --learning-rate-step-unit epochs --gamma 0.1 \
        --N 2 --training-unit epochs

Multi-GPU: ``python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train.py ...``.
Data: ``--metadata <file>`` of a binary data set written by ``DatasetWriter``, or, as the reference's applications take it
(ResNetv1ForCifar.java:797-1029, ResNetv1.java:861-1091, VGG.java:377-513), ``--dataset-name cifar-10|cifar-100|mnist|imagenet
--data-directory <dir>`` holding ``<alias>-train.metadata`` / ``<alias>-test.metadata`` (ImageNet: ``crossbow-train.records.*``
record files of JPEGs are used when the directory has them); without either a synthetic data set of the model's input shape
is generated.  ``--model resnet --layers 50`` picks the depth; ``--time-limit true --D 30 --duration-unit minutes`` trains
for a duration instead of ``--N`` units; ``--unit`` is an alias of ``--training-unit``; ``--weight-initialiser constant|gaussian`` overrides the initialisers of the
convolution and inner-product layers.
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
    # the flags of the reference's applications
    opts.add(Option("--layers", int, 0)).add(Option("--dataset-name", str, None)).add(Option("--data-directory", str, None))
    opts.add(Option("--time-limit", str, "false")).add(Option("--D", float, 1.0)).add(Option("--duration-unit", str, "minutes"))
    opts.add(Option("--unit", str, None)).add(Option("--weight-initialiser", str, None))
    CommandLine(opts).parse(argv)
    sysc, mc = SystemConf.getInstance(), ModelConf.getInstance()
    name, layers, dataset = opts.get("--model").get(), opts.get("--layers").get(), opts.get("--dataset-name").get()
    if name in ("resnet", "resnetv1"):                # depth and data set pick the network, as in ResNetv1ForCifar.java:888-960
        layers = layers or (50 if dataset == "imagenet" else 32)
        if dataset == "imagenet" and layers not in (18, 34, 50, 101, 152) or dataset != "imagenet" and (layers - 2) % 6:
            raise SystemExit(f"error: invalid number of layers for {dataset or 'cifar-10'} dataset")
        name = f"resnet{layers}"
    spec = build(name, solver_conf=mc.getSolverConf())
    wi = opts.get("--weight-initialiser").get()
    if wi:                                            # LeNetBatchNorm.java:118-139, ConvNet.java: constant (0, bias 1) or gaussian (std 0.1, bias 0)
        from crossbow_b200 import InitialiserConf, InitialiserType
        kind = InitialiserType.from_string(wi)
        if kind not in (InitialiserType.CONSTANT, InitialiserType.GAUSSIAN):
            raise SystemExit("error: weight initialiser must be either constant or gaussian")
        for g in (spec.train, spec.test):
            for node in (g.nodes() if g is not None else []):
                k = node.op.kernel
                if getattr(k, "kind", "") in ("conv", "innerproduct") and not k.is_gradient:
                    if kind == InitialiserType.CONSTANT:
                        k.conf.setWeightInitialiser(InitialiserConf().setType(kind).setValue(0)).setBiasInitialiser(InitialiserConf().setType(kind).setValue(1))
                    else:
                        k.conf.setWeightInitialiser(InitialiserConf().setType(kind).setStd(0.1))
                        k.conf.setBiasInitialiser(InitialiserConf().setType(InitialiserType.CONSTANT).setValue(0))
    if int(os.environ.get("WORLD_SIZE", 1)) > 1:      # one process per GPU (nccl) or per CPU device group (gloo)
        from crossbow_b200.parallel.peer import init_process_group
        init_process_group()
    directory = opts.get("--data-directory").get()
    if dataset and directory and not opts.get("--metadata").get():
        import glob
        alias = {"cifar-10": "cifar", "cifar-100": "cifar", "mnist": "mnist", "imagenet": "imagenet"}.get(dataset, dataset)
        records = sorted(glob.glob(os.path.join(directory, "crossbow-train.records.*")))
        if records:                                   # JPEG record files (RecordDataset.java:59-99)
            from crossbow_b200.data.records import RecordDataset
            size = spec.input_shape[-1]
            train = RecordDataset(records, mc.batch_size, image_size=size, workers=max(1, sysc.number_of_file_handlers), training=True,
                                  seed=sysc.random_seed, register_with_cuda=sysc.gpu)
            held = sorted(glob.glob(os.path.join(directory, "crossbow-validation.records.*")))
            test = RecordDataset(held, mc.batch_size, image_size=size, workers=max(1, sysc.number_of_file_handlers), training=False,
                                 register_with_cuda=sysc.gpu) if held else None
        else:
            opts.get("--metadata").set(os.path.join(directory, f"{alias}-train.metadata"))
            if os.path.exists(os.path.join(directory, f"{alias}-test.metadata")):
                opts.get("--test-metadata").set(os.path.join(directory, f"{alias}-test.metadata"))
    if dataset and directory and not opts.get("--metadata").get():
        pass                                          # record files: the data sets are open
    elif opts.get("--metadata").get():
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
    n, unit = opts.get("--N").get(), TrainingUnit.from_string(opts.get("--unit").get() or opts.get("--training-unit").get())
    if str(opts.get("--time-limit").get()).lower() in ("true", "1", "yes"):
        from crossbow_b200 import DurationUnit
        d, du = opts.get("--D").get(), DurationUnit.from_string(opts.get("--duration-unit").get())
        if opts.get("--target-loss").get() > 0:
            ctx.trainUntilConditionOrForDuration(opts.get("--target-loss").get(), d, du)
        else:
            ctx.trainForDuration(d, du)
    elif opts.get("--target-loss").get() > 0:
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

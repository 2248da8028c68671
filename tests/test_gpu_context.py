"""ExecutionContext on the GPU through the native scheduler: training, testing, auto-tuning, checkpoint / resume,
binary data sets feeding the scheduler directly."""
import os

import numpy as np
import pytest
import torch

from crossbow_b200 import Dataflow, ModelConf, Phase, SystemConf, UpdateModel
from crossbow_b200.context import ExecutionContext
from crossbow_b200.data import SyntheticDataset
from crossbow_b200.models import build

pytestmark = pytest.mark.gpu


def _context(model="lenet-caffe", shape=(1, 28, 28), k=2, batch=16, update="SMA", autotune=False, lr=0.01, batches=8, **sys_kw):
    sysc, mc = SystemConf.reset(), ModelConf.reset()
    sysc.setGPU(True).setCPU(False).setNumberOfGpuModels(k).setDisplayInterval(0)
    sysc.autotune_models = autotune
    for key, v in sys_kw.items():
        setattr(sysc, key, v)
    solver = mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(lr).setMomentum(0.9).setAlpha(0.1)
    mc.setBatchSize(batch).setWpc(k).setUpdateModel(update)
    ds = SyntheticDataset(list(shape), 10, batch, batches=batches, seed=1, distribution="uniform")
    mc.setDataset(Phase.TRAIN, ds).setDataset(Phase.CHECK, ds)
    spec = build(model, solver_conf=solver)
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), Dataflow(spec.test).setPhase(Phase.CHECK)], quiet=True)
    ctx.init()
    return ctx


@pytest.mark.parametrize("native", [True, False])
def test_train_test_and_loss_goes_down(native):
    ctx = _context(native_scheduler=native)
    assert (ctx._native is not None) == native
    ctx.train(64, "tasks")
    losses = ctx.measurements.losses()
    assert len(losses) == 64 and np.isfinite(losses).all()
    assert np.mean(losses[-8:]) < np.mean(losses[:8])          # 8 distinct batches, seen 8 times each
    acc = ctx.test()
    assert 0.0 <= acc <= 1.0
    assert ctx.clock.clock == 32
    ctx.destroy()


def test_synchronous_sgd_with_gradient_buckets_through_the_native_scheduler():
    ref = _context(update="WORKER", gradient_buckets=1)
    ref.train(16, "tasks")
    z1 = ref.engine.central_model()
    ref.destroy()
    ctx = _context(update="WORKER", gradient_buckets=3)
    assert ctx._native is not None and len(ctx.engine.bucket_syncs) >= 2
    ctx.train(16, "tasks")
    z2 = ctx.engine.central_model()
    losses = ctx.measurements.losses()
    ctx.destroy()
    assert np.isfinite(losses).all()
    # same arithmetic, different launch boundaries: the runs differ only through the order of the fp32 atomic additions in
    # the split reductions (weight gradients, batch-sized inner products), which 16 steps of momentum amplify a little
    assert np.abs(z1 - z2).max() <= 3e-4 * np.abs(z1).max()


def test_tracing_collects_task_times_and_makespan():
    from crossbow_b200.utils import trace
    ctx = _context(trace_level=2, use_cuda_graphs=False)           # per-operator NVTX ranges are issued with every eager launch
    try:
        assert trace.level() == 2
        ctx.train(16, "tasks")
        dev, gaps = trace.task_device_ms(), trace.inter_arrival_us()
        assert len(dev) == 16 and (dev > 0).all() and len(gaps) == 15 and (gaps > 0).all()
        st = trace.summary()
        assert st["task_device_ms"]["p50"] <= st["task_device_ms"]["max"]
        ms = trace.makespan_ms(ctx.engine, tasks_per_learner=3, park_ms=5.0)
        # the tasks were all queued behind the sleep kernels: the makespan covers at least one task's device time
        assert ms >= float(dev.min()) * 0.5 and ms < 5000
    finally:
        ctx.destroy()
    assert trace.level() == 0 and ctx.trace_summary["task_device_ms"]["n"] >= 16


def test_checkpoint_and_resume(tmp_path):
    ctx = _context()
    ctx.train(8, "tasks")
    d = ctx.checkpoint(str(tmp_path))
    z = ctx.engine.central_model()
    r1 = ctx.engine.replica_model(1)
    assert os.path.getsize(os.path.join(d, "gpu-00-theModel-data.dat")) == 4 * ctx.model.elements
    assert os.path.exists(os.path.join(d, "gpu-00-replica-001-last.dat"))
    ctx.destroy()
    ctx2 = _context(model_directory=str(tmp_path))
    assert np.array_equal(ctx2.engine.central_model(), z) and np.array_equal(ctx2.engine.replica_model(1), r1)
    ctx2.train(4, "tasks")
    ctx2.destroy()


def test_batch_norm_statistics_are_checkpointed(tmp_path):
    ctx = _context(model="resnet8", shape=(3, 32, 32), batch=8)
    ctx.train(4, "tasks")
    d = ctx.checkpoint(str(tmp_path))
    assert any(f.startswith("gpu-00-bn-avg-") for f in os.listdir(d)) and any(f.startswith("gpu-00-bn-var-") for f in os.listdir(d))
    ctx.destroy()


def test_auto_tuner_adds_and_removes_replicas():
    ctx = _context(k=1, autotune=True, autotune_threshold=-1.0, monitor_interval=1)   # any throughput counts as an improvement -> keeps adding
    ctx.train(24, "tasks")
    assert ctx.engine.k > 1
    k = ctx.engine.k
    ctx.autotuner.threshold = 1e9                                   # nothing improves by that much -> remove one and stop
    ctx.train(16, "tasks")
    assert ctx.engine.k == k - 1 and not ctx.autotuner.active
    assert np.isfinite(ctx.measurements.losses()).all()
    ctx.destroy()


def test_auto_tuner_finds_the_knee_of_resnet32():
    """`--autotune-models true` with the default threshold (0.1) on the headline workload, starting from one replica: the
    tuner must climb while throughput rises by more than 10 % per added replica, stop for good at the first sample that
    does not and step back by one; throughput measured at fixed replica counts in the same context must agree with what it
    decided.  (12 tasks per clock, so that one to four replicas all divide a clock evenly.)"""
    import time
    sysc, mc = SystemConf.reset(), ModelConf.reset()
    sysc.setGPU(True).setCPU(False).setNumberOfGpuModels(1).setDisplayInterval(0)
    sysc.autotune_models, sysc.monitor_interval = True, 300
    assert sysc.autotune_threshold == 0.1 and sysc.autotune_interval == 1
    solver = mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.01).setMomentum(0.9).setAlpha(0.1).setWeightDecay(1e-4)
    mc.setBatchSize(64).setWpc(12).setUpdateModel("SMA")
    mc.setDataset(Phase.TRAIN, SyntheticDataset([3, 32, 32], 10, 64, batches=24, seed=1))
    spec = build("resnet32", solver_conf=solver)
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), None], quiet=True)
    ctx.init()
    try:
        assert ctx._native is not None
        ctx.train(48, "tasks")                                      # warm-up without a decision (shorter than one interval)
        for _ in range(40):
            if not ctx.autotuner.active:
                break
            ctx.train(480, "tasks")
        trace = list(ctx.autotune_trace)
        print("auto-tuner trace (replicas after the decision, job examples/s it was based on):", [(k, round(r)) for k, r in trace])
        print("chunks while tuning (replicas, tasks, ms, settling):", [(k, n, round(dt * 1e3, 1), st) for k, n, dt, st in ctx.autotune_chunks])
        assert not ctx.autotuner.active, "the tuner never stopped"
        k_final = ctx.engine.k
        ks = [k for k, _ in trace]
        samples = [r for _, r in trace]
        assert k_final >= 2 and ks == list(range(2, k_final + 2)) + [k_final]       # climbed one by one, overshot by one, stepped back
        assert all(b > 1.1 * a for a, b in zip(samples[:-2], samples[1:-1]))        # every step it kept had brought more than 10 %
        assert samples[-1] <= 1.1 * samples[-2]                                     # the one it undid had not
        # throughput at fixed replica counts, same context: what the samples claimed must hold there too
        rates = {}

        def rate():
            ctx.train(48, "tasks")
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            n = ctx.train(480, "tasks")
            return n * 64 / (time.perf_counter() - t0)
        rates[k_final] = rate()
        for k in range(k_final + 1, k_final + 3):
            ctx.engine.add_learner()
            ctx._native.add_learner()
            rates[k] = rate()
        print("fixed replica counts:", {k: round(v) for k, v in rates.items()}, "tuner stopped at", k_final)
        assert rates[k_final] > 1.3 * samples[0]                                    # well above one replica
        assert rates[k_final + 1] < 1.15 * rates[k_final]                           # and the next replica is indeed not worth 10 % (5 % slack)
        assert np.isfinite(ctx.measurements.losses()).all()
    finally:
        ctx.destroy()


def test_binary_dataset_feeds_the_scheduler(tmp_path):
    from crossbow_b200.data.native import DatasetWriter, LightDataset
    g = np.random.default_rng(0)
    w = DatasetWriter(str(tmp_path), "toy", (1, 28, 28), 16)
    w.append(g.random((64, 1, 28, 28), dtype=np.float32), g.integers(0, 10, 64))
    meta = w.close()
    sysc, mc = SystemConf.reset(), ModelConf.reset()
    sysc.setGPU(True).setCPU(False).setNumberOfGpuModels(2).setDisplayInterval(0)
    solver = mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.01).setMomentum(0.9).setAlpha(0.1)
    mc.setBatchSize(16).setWpc(2).setUpdateModel("SMA")
    ds = LightDataset(meta, slots=4, copiers=1, register_with_cuda=True)
    mc.setDataset(Phase.TRAIN, ds)
    spec = build("lenet-caffe", solver_conf=solver)
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), None], quiet=True)
    ctx.init()
    assert ctx._native is not None       # the C++ scheduler pulls batches straight from the C++ slot ring
    ctx.train(12, "tasks")
    assert len(ctx.measurements.losses()) == 12 and np.isfinite(ctx.measurements.losses()).all()
    ctx.destroy()
    ds.close()

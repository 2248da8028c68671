"""Host-only tests: configuration, CLI parsing, schedules, initialisers, graph construction, oracle, sync maths,
checkpoint layout, clock / auto-tuner, counter-based RNG."""
import math
import os

import numpy as np
import pytest
import torch

from crossbow_b200 import *  # noqa: F401,F403
from crossbow_b200.autotune import AutoTuner
from crossbow_b200.kernels import OpEnv, pool_output_size
from crossbow_b200.models import build
from crossbow_b200.oracle import (DeviceState, OracleExecutor, ReplicaState, local_update, synchronise_sma,
                                  synchronise_ssgd, synchronise_polyak_ruppert, synchronise_eamsgd)
from crossbow_b200.utils.philox import philox4x32, philox_uniform
from crossbow_b200.workclock import WorkClock
from helpers import build_model, make_batches, make_solver


def test_philox_known_answers():
    o = philox4x32([0], [0], [0], [0], 0, 0)
    assert [int(x[0]) for x in o] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    o = philox4x32([0xFFFFFFFF] * 1, [0xFFFFFFFF], [0xFFFFFFFF], [0xFFFFFFFF], 0xFFFFFFFF, 0xFFFFFFFF)
    assert [int(x[0]) for x in o] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    u = philox_uniform(10001, 42, 3, 9)
    assert u.min() >= 0 and u.max() < 1 and abs(u.mean() - 0.5) < 0.02
    assert np.array_equal(u[:100], philox_uniform(100, 42, 3, 9))


def test_system_and_model_conf_parse_all_flags():
    s, m = SystemConf.reset(), ModelConf.reset()
    flags = {"--gpu": "true", "--gpu-devices": "0,1,2,3", "--number-of-gpu-models": "4", "--synchronisation-model": "SSP",
             "--autotune-models": "true", "--autotune-threshold": "0.2", "--task-queue-size": "64", "--random-seed": "7",
             "--scheduling-policy": "FIFO", "--display-interval-unit": "epochs"}
    for k, v in flags.items():
        assert s.parse(k, v), k
    assert s.gpu and s.gpu_devices == [0, 1, 2, 3] and s.number_of_gpu_models == 4
    assert s.synchronisation_model == SynchronisationModel.SSP and s.autotune_threshold == 0.2
    assert s.numberOfGPUs() == 4 and s.getNumberOfGpuModels() == 4
    assert len(SystemConf.OPTIONS) >= 37
    for k, v in {"--wpc": "8", "--slack": "1", "--batch-size": "64", "--update-model": "SMA", "--learning-rate": "0.1",
                 "--momentum": "0.9", "--step-values": "80,120", "--learning-rate-decay-policy": "multistep", "--alpha": "0.1"}.items():
        assert m.parse(k, v), k
    assert m.wpc == 8 and m.update_model == UpdateModel.SMA and m.getSolverConf().step_values == [80, 120]
    assert not m.parse("--no-such-flag", "1")


def test_fluent_setters_match_reference_spelling():
    c = ConvConf().setNumberOfOutputs(32).setKernelSize(2).setKernelHeight(5).setKernelWidth(5).setBias(False)
    assert (c.number_of_outputs, c.kernel_height, c.kernel_width, c.bias) == (32, 5, 5, False)
    p = PoolConf().setKernelSize(2).setStrideSize(2).setPaddingSize(0)
    assert (p.kernel_height, p.stride_width) == (2, 2)
    b = BatchNormConf().setEpsilon(1e-5).setMovingAverageFraction(0.9)
    assert b.fraction == 0.9
    i = InitialiserConf().setType(InitialiserType.GAUSSIAN).setStd(0.1).truncate(True)
    assert i.type == InitialiserType.GAUSSIAN and i.truncated


def test_learning_rate_schedules():
    s = SolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.1)
    assert s.learning_rate(5) == pytest.approx(0.1)
    s = SolverConf().setLearningRateDecayPolicy("INV").setBaseLearningRate(0.1).setGamma(0.001).setPower(0.75)
    assert s.learning_rate(9) == pytest.approx(0.1 * (1 + 0.001 * 10) ** -0.75)
    s = SolverConf().setLearningRateDecayPolicy("STEP").setBaseLearningRate(1.0).setGamma(0.5).setStepSize(10)
    assert s.learning_rate(8) == 1.0 and s.learning_rate(9) == 0.5 and s.learning_rate(19) == 0.25
    s = SolverConf().setLearningRateDecayPolicy("EXP").setBaseLearningRate(1.0).setGamma(0.9)
    assert s.learning_rate(1) == pytest.approx(0.81)
    s = SolverConf().setLearningRateDecayPolicy("MULTISTEP").setBaseLearningRate(1.0).setGamma(0.1).setStepValues(3, 5)
    rates = [s.learning_rate(t) for t in range(6)]
    assert rates[:2] == [1.0, 1.0] and rates[2] == pytest.approx(0.1) and rates[4] == pytest.approx(0.01)
    assert s.consume_copy_signal() and not s.consume_copy_signal()
    s = SolverConf().setLearningRateDecayPolicy("LSR").setBaseLearningRate(1.0).setGamma(0.1).setStepValues(10).setWarmupSteps(4)
    assert [s.learning_rate(t) for t in range(4)] == [0.0, 0.25, 0.5, 0.75] and s.learning_rate(4) == 1.0
    s = SolverConf().setLearningRateDecayPolicy("MULTISTEP").setBaseLearningRate(1.0).setGamma(0.1).setStepValues(2)
    s.step_unit = TrainingUnit.EPOCHS
    s.set_tasks_per_epoch(10)
    assert s.learning_rate(18) == 1.0 and s.learning_rate(19) == pytest.approx(0.1)


def test_initialisers():
    m = Model()
    spec, m, _ = build_model("lenet", 4)
    w = m.initial_values(123)
    assert w.shape == (m.elements,) and np.isfinite(w).all()
    conv = m.variables[0]
    vals = w[conv.offset:conv.offset + conv.elements()]
    assert abs(vals.std() - 0.1) < 0.03 and np.abs(vals).max() <= 0.2 + 1e-6        # truncated at 2 sigma
    assert np.array_equal(w, m.initial_values(123)) and not np.array_equal(w, m.initial_values(124))
    v = Variable("w", Shape([8, 4, 3, 3])).initialise(InitialiserConf().setType("XAVIER"))
    from crossbow_b200.model import RandomGenerator
    x = v.generate(RandomGenerator(1))
    assert np.abs(x).max() <= math.sqrt(3.0 / 36) + 1e-6
    v.initialise(InitialiserConf().setType("MSRA"))
    assert abs(v.generate(RandomGenerator(1)).std() - math.sqrt(2.0 / 72)) < 0.03


def test_device_layout_roundtrip():
    spec, m, _ = build_model("lenet", 4)
    w = m.initial_values(5)
    d = m.to_device(w)
    assert d.size == m.device_elements and m.device_elements % 64 == 0
    assert all(v.doffset % 64 == 0 for v in m.variables)
    assert np.array_equal(m.to_canonical(d), w)
    conv = m.variables[0]
    K, Cc, R, S = conv.shape.dims
    a = w[conv.offset:conv.offset + conv.elements()].reshape(K, Cc, R, S)
    b = d[conv.doffset:conv.doffset + conv.elements()].reshape(K, R, S, Cc)
    assert np.array_equal(a.transpose(0, 2, 3, 1), b)


def test_pool_ceil_mode_shapes():
    assert pool_output_size(112, 3, 2, 0) == 56
    assert pool_output_size(112, 3, 2, 1) == 57
    assert pool_output_size(32, 2, 2, 0) == 16
    assert pool_output_size(7, 3, 2, 1) == 4
    assert pool_output_size(8, 7, 1, 0) == 2


def test_graph_api_manual_gradient_chain():
    """The reference's explicit style: forward chain, gradient nodes with peers, optimiser."""
    ip = InnerProductConf().setNumberOfOutputs(10)
    ip.setWeightInitialiser(InitialiserConf().setType("GAUSSIAN").setStd(0.1))
    lc = LossConf()
    n_ip = DataflowNode(Operator("InnerProduct", InnerProduct(ip)))
    n_sm = DataflowNode(Operator("SoftMax", SoftMax(SoftMaxConf())))
    n_loss = DataflowNode(Operator("Loss", SoftMaxLoss(lc)))
    n_acc = DataflowNode(Operator("Accuracy", Accuracy(AccuracyConf())))
    n_lg = DataflowNode(Operator("LossGradient", SoftMaxLossGradient(lc)).setPeer(n_loss.getOperator()))
    n_ig = DataflowNode(Operator("InnerProductGradient", InnerProductGradient(ip)).setPeer(n_ip.getOperator()))
    n_opt = DataflowNode(Operator("Optimiser", GradientDescentOptimiser(make_solver())))
    n_ip.connectTo(n_sm).connectTo(n_loss)
    n_sm.connectTo(n_acc)
    n_loss.connectTo(n_lg).connectTo(n_ig).connectTo(n_opt)
    g = SubGraph(n_ip)
    m = Model()
    g.init(Shape([4, 20, 1, 1]), Shape([4]), m)
    m.finalise()
    names = [n.op.name for n in g.order]
    assert names.index("InnerProduct") < names.index("SoftMax") < names.index("Loss") < names.index("LossGradient") < names.index("Optimiser")
    assert m.elements == 20 * 10 + 10
    w = torch.from_numpy(m.initial_values(1))
    x, y = torch.randn(4, 20, 1, 1), torch.tensor([1, 2, 3, 4], dtype=torch.int32)
    grad = torch.zeros_like(w)
    r = OracleExecutor(g, m).run(w, x, y, Phase.TRAIN, grad_out=grad)
    wp = w.clone().requires_grad_(True)
    logits = torch.nn.functional.linear(x.reshape(4, -1), wp[:200].reshape(10, 20), wp[200:])
    loss = torch.nn.functional.cross_entropy(logits, y.long())
    loss.backward()
    assert r["loss"] == pytest.approx(float(loss), rel=1e-5)
    assert torch.allclose(grad, wp.grad, atol=1e-6)
    assert "digraph" in g.exportDot()
    df = Dataflow(g).setPhase(Phase.TRAIN)
    assert df.getPhase() == Phase.TRAIN and "InnerProduct" in df.dump()


@pytest.mark.parametrize("name", ["resnet8", "mini-inception", "lenet-batchnorm"])
def test_oracle_gradients_equal_monolithic_autograd(name):
    spec, m, _ = build_model(name, 4)
    w = torch.from_numpy(m.initial_values(1))
    xs, ys = make_batches(spec, 4, 1)
    grad = torch.zeros_like(w)
    r = OracleExecutor(spec.train, m, seed=1).run(w, xs[0], ys[0], Phase.TRAIN, 0, {}, grad)
    wp = w.clone().requires_grad_(True)
    env = OpEnv(Phase.TRAIN, ys[0], 0, 1, {})
    outs = {}
    for node in spec.train.order:
        k = node.op.kernel
        if k.is_gradient or k.is_optimiser or getattr(k, "is_gradient_merge", False):
            continue
        ins = [outs[id(p)] for p in node.prev if not p.op.kernel.is_gradient] or [xs[0]]
        params = [wp[v.offset:v.offset + v.elements()].reshape(v.shape.dims) for v in k.variables]
        outs[id(node)] = k.forward(ins, params, env)
        if k.is_loss:
            loss = outs[id(node)]
    loss.sum().backward()
    assert r["loss"] == pytest.approx(float(loss.detach()), rel=1e-5)
    assert torch.allclose(grad, wp.grad, atol=2e-6, rtol=1e-4)


def test_test_graph_shares_operators_and_drops_dropout():
    spec, m, _ = build_model("lenet", 4)
    train_ops = {n.op.uid for n in spec.train.order}
    assert all(n.op.uid in train_ops for n in spec.test.order)
    assert not any(n.op.kernel.kind == "dropout" for n in spec.test.order)
    assert any(n.op.kernel.kind == "accuracy" for n in spec.test.order)


def _devs(G, k, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    base = torch.randn(n, generator=g)
    out = []
    for _ in range(G):
        d = DeviceState(base)
        for _ in range(k):
            r = ReplicaState(base + 0.1 * torch.randn(n, generator=g))
            r.prev = r.w.clone()
            d.replicas.append(r)
        out.append(d)
    return out


def test_sma_keeps_devices_identical_and_moves_towards_mean():
    devs = _devs(2, 2, 50)
    mean_before = sum(r.w for d in devs for r in d.replicas) / 4
    z_before = devs[0].z.clone()
    synchronise_sma(devs, 0.25, 0.0)
    assert torch.equal(devs[0].z, devs[1].z)
    assert torch.allclose(devs[0].z, z_before + 0.25 * 4 * (mean_before - z_before), atol=1e-5)


def test_sma_copy_on_rate_drop():
    devs = _devs(1, 2, 10)
    synchronise_sma(devs, 0.1, 0.9, copy=True)
    assert all(torch.equal(r.w, devs[0].z) for r in devs[0].replicas)


def test_ssgd_equals_large_batch_sgd():
    n = 20
    devs = _devs(2, 2, n)
    s = make_solver(lr=0.1, momentum=0.0, wd=0.0)
    grads = [torch.randn(n) for _ in range(4)]
    z0 = devs[0].z.clone()
    i = 0
    for d in devs:
        for r in d.replicas:
            r.g = grads[i].clone()
            local_update(r, d, s, UpdateModel.WORKER, 0)
            i += 1
    synchronise_ssgd(devs, 4, 0.0)
    assert torch.allclose(devs[0].z, z0 - 0.1 * sum(grads) / 4, atol=1e-6)
    assert all(torch.equal(r.w, d.z) for d in devs for r in d.replicas)


def test_local_update_momentum_and_snapshot():
    d = DeviceState(torch.ones(4))
    r = ReplicaState(torch.ones(4))
    s = make_solver(lr=0.5, momentum=0.9, wd=0.0)
    r.g = torch.full((4,), 2.0)
    local_update(r, d, s, UpdateModel.SMA, 0)
    assert torch.allclose(r.prev, torch.ones(4)) and torch.allclose(r.w, torch.zeros(4)) and torch.allclose(r.last, -torch.ones(4))
    r.g = torch.full((4,), 2.0)
    local_update(r, d, s, UpdateModel.SMA, 1)
    assert torch.allclose(r.w, torch.full((4,), -1.9))
    s2 = make_solver(lr=1.0, momentum=0.0, wd=0.0).setClipGradientThreshold(1.0)
    r2 = ReplicaState(torch.zeros(4))
    r2.g = torch.full((4,), 3.0)
    local_update(r2, d, s2, UpdateModel.SMA, 0)
    assert torch.allclose(r2.w, torch.full((4,), -0.5))


def test_polyak_and_eamsgd():
    devs = _devs(1, 2, 8)
    mean = sum(r.w for r in devs[0].replicas) / 2
    synchronise_polyak_ruppert(devs)
    assert torch.allclose(devs[0].z, mean)
    devs = _devs(1, 2, 8)
    w0 = [r.w.clone() for r in devs[0].replicas]
    z0 = devs[0].z.clone()
    synchronise_eamsgd(devs, 0.5)
    assert torch.allclose(devs[0].replicas[0].w, w0[0] - 0.5 * (w0[0] - z0))


def test_work_clock_and_autotuner():
    c = WorkClock(3)
    seen = []
    for _ in range(7):
        t = c.next_task()
        if c.is_barrier():
            c.tick()
            seen.append(t)
    assert seen == [2, 5] and c.clock == 2 and c.lower_bound(1) == 0
    a = AutoTuner(0.1, 1)
    assert a.decide([100.0]) == 1 and a.decide([100.0, 150.0]) == 1 and a.decide([150.0, 155.0]) == -1
    assert a.decide([400.0]) == 0 and not a.active


def test_cpu_context_trains_lenet_sma_and_checkpoints(tmp_path):
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.data import SyntheticDataset
    SystemConf.reset().setNumberOfCpuModels(2).setDisplayInterval(0)
    mc = ModelConf.reset()
    sc = mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.01).setMomentum(0.9).setAlpha(0.1)
    mc.setBatchSize(16).setWpc(2).setUpdateModel("SMA")
    ds = SyntheticDataset([1, 28, 28], 10, 16, batches=2, seed=1, distribution="uniform")
    mc.setDataset(Phase.TRAIN, ds).setDataset(Phase.CHECK, ds)
    spec = build("lenet-caffe", solver_conf=sc)
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), Dataflow(spec.test).setPhase(Phase.CHECK)], quiet=True)
    ctx.init()
    ctx.train(16, "tasks")
    losses = ctx.measurements.losses()
    assert len(losses) == 16 and np.mean(losses[-4:]) < np.mean(losses[:4])
    acc = ctx.test()
    assert 0.0 <= acc <= 1.0
    d = ctx.checkpoint(str(tmp_path))
    files = sorted(os.listdir(d))
    assert files == ["gpu-00-replica-000-data.dat", "gpu-00-replica-000-last.dat", "gpu-00-replica-001-data.dat",
                     "gpu-00-replica-001-last.dat", "gpu-00-theModel-data.dat", "gpu-00-theModel-last.dat"]
    assert os.path.getsize(os.path.join(d, files[4])) == 4 * ctx.model.elements
    z = ctx.engine.central_model()
    # resume into a fresh context
    SystemConf.getInstance().setModelDirectory(str(tmp_path))
    spec2 = build("lenet-caffe", solver_conf=sc)
    ctx2 = ExecutionContext([Dataflow(spec2.train).setPhase(Phase.TRAIN), Dataflow(spec2.test).setPhase(Phase.CHECK)], quiet=True)
    ctx2.init()
    assert np.array_equal(ctx2.engine.central_model(), z)
    assert np.array_equal(ctx2.engine.replica_model(1), ctx.engine.replica_model(1))


def test_all_models_build_and_infer_shapes():
    from crossbow_b200.models import REGISTRY
    sizes = {"resnet18": 64, "resnet34": 64, "resnet50": 64, "resnet101": 64, "resnet152": 64, "alexnet": 224, "overfeat": 231,
             "vgg-a": 64}
    for name in REGISTRY:
        kw = {"size": sizes[name]} if name in sizes else {}
        spec, m, _ = build_model(name, 2, **kw)
        assert m.elements > 0 and spec.train.getLossNode() is not None
        assert spec.test is None or spec.test.getAccuracyNode() is not None      # (matrix factorisation has no test graph)
    spec, m, _ = build_model("resnet32", 2)
    assert 460000 < m.elements < 470000
    # any CIFAR depth 6n + 2 builds (ResNetv1ForCifar.java:952-960), anything else is refused
    from crossbow_b200.models import build as build_spec
    assert build_spec("resnet14").name == "resnet-14" and build_spec("baby-resnet").name == "resnet-8"
    with pytest.raises(ValueError):
        build_spec("resnet15")
    spec, m, _ = build_model("resnet50", 2, size=224)
    assert 25.5e6 < m.elements < 25.7e6


def test_batch_splits_equal_consecutive_sub_batch_tasks():
    """A task of 8 examples with 2 splits = two updates on its halves (taskhandler.c:65-114 slides the input window)."""
    from crossbow_b200.engine import CpuEngine
    import copy
    spec, m, solver = build_model("mlp", 8)
    init = m.initial_values(3)
    xs, ys = make_batches(spec, 8, 2, seed=4)
    a = CpuEngine(spec.train, spec.test, m, init, 8, spec.input_shape, copy.deepcopy(solver), UpdateModel.DEFAULT, splits=2)
    b = CpuEngine(spec.train, spec.test, m, init, 4, spec.input_shape, copy.deepcopy(solver), UpdateModel.DEFAULT)
    for t in range(2):
        a.submit(0, xs[t], ys[t], t)
        la, _ = a.wait(0)
        lb = []
        for s in range(2):
            b.submit(0, xs[t][4 * s:4 * s + 4], ys[t][4 * s:4 * s + 4], t)
            lb.append(b.wait(0)[0])
        assert la == pytest.approx(sum(lb) / 2, rel=1e-6)
    assert np.allclose(a.replica_model(0), b.replica_model(0), rtol=1e-6, atol=1e-7)


def test_matmul_is_an_inner_product_without_bias():
    from crossbow_b200.conf import InnerProductConf
    from crossbow_b200.kernels import MatMul
    m = Model()
    k = MatMul(InnerProductConf().setNumberOfOutputs(5))
    node = DataflowNode(Operator("MatMul", k))
    g = SubGraph(node)
    g.init(Shape([3, 7]), Shape([3]), m)
    m.finalise()
    assert [v.name for v in k.variables] == ["weights"] and m.elements == 35
    w = torch.from_numpy(m.initial_values(1)).reshape(5, 7)
    x = torch.randn(3, 7)
    assert torch.allclose(k.forward([x], [w], None), x @ w.t())


def test_display_interval_accumulated_loss_queue_and_tee(capsys):
    """Display semantics of the training result handler: interval, accumulated mean, queued records, tee."""
    from crossbow_b200.context import ExecutionContext
    ctx = ExecutionContext.__new__(ExecutionContext)
    from crossbow_b200.utils.measure import MeasurementQueue, PerformanceMonitor
    sysc = SystemConf.reset()
    ctx.sys, ctx.quiet = sysc, False
    ctx.displayed, ctx.monitor = MeasurementQueue(), PerformanceMonitor(8, 0)
    ctx._disp_n, ctx._disp_loss, ctx._disp_acc = 0, 0.0, 0.0
    sysc.display_interval, sysc.display_accumulated_loss = 2, True
    for t, (l, a) in enumerate([(4.0, 0.0), (2.0, 1.0), (1.0, 0.5), (3.0, 0.5)]):
        ctx._display(t, l, a)
    out = capsys.readouterr().out.splitlines()
    assert len(out) == 2 and "loss   3.00000 (  2.00000)" in out[0] and "accuracy  0.5000 ( 1.0000)" in out[0] and "[000004]" in out[1]
    sysc.display_accumulated_loss, sysc.queue_measurements, sysc.tee_measurements = False, True, False
    ctx._display(4, 9.0, 0.0)
    ctx._display(5, 7.0, 0.25)
    assert capsys.readouterr().out == "" and len(ctx.displayed) == 1 and ctx.displayed.losses() == [7.0]
    sysc.tee_measurements = True
    ctx._display(6, 1.0, 0.0)
    ctx._display(7, 0.5, 1.0)
    assert "loss   0.50000 accuracy  1.0000" in capsys.readouterr().out and len(ctx.displayed) == 2


def test_trace_percentiles_and_gpu_sampler_summary():
    from crossbow_b200.utils.trace import percentiles
    st = percentiles(np.arange(1, 101, dtype=np.float32))
    assert st["n"] == 100 and st["min"] == 1 and st["max"] == 100 and abs(st["p50"] - 50.5) < 1e-3 and abs(st["p99"] - 99.01) < 1e-2
    assert percentiles(np.array([])) == {"n": 0}


def test_execution_context_accessors():
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.data import SyntheticDataset
    from crossbow_b200.models import build
    sysc, mc = SystemConf.reset(), ModelConf.reset()
    sysc.setCPU(True).setGPU(False).setDisplayInterval(0)
    solver = mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.01)
    mc.setBatchSize(8).setWpc(1).setUpdateModel("SMA")
    mc.setDataset(Phase.TRAIN, SyntheticDataset([1, 28, 28], 10, 8, batches=4, seed=1, distribution="uniform"))
    spec = build("logistic-regression", solver_conf=solver)
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), None], quiet=True)
    ctx.init()
    ctx.train(4, "tasks")
    assert len(ctx.getDataflows()) == 2 and ctx.getDataflow("TRAIN") is ctx.dataflows[0] and ctx.getDataflow(Phase.CHECK) is None
    assert ctx.getModel().elements == 7850 and ctx.getWorkClock().clock == 4 and ctx.getExecutorQueueSize() == 0
    m = ctx.getThroughputMatrix()
    assert len(m) == 2 and len(m[0]) == 2 and m[1] == [0, 0]           # CPU row measured, GPU row empty
    assert ctx.getModelManager() is ctx.engine
    ctx.destroy()


def test_reference_setter_names_exist():
    """A program written against the reference's configuration API keeps working (SystemConf.java, ModelConf.java, SolverConf.java)."""
    s = SystemConf.reset().setCPU(False).setGPU(True).setGPUDevices(0, 1).setNumberOfWorkerThreads(1).setNumberOfCPUModelReplicas(1) \
        .setNumberOfReadersPerModel(1).setNumberOfGPUModelReplicas(3).setNumberOfGPUStreams(3).setNumberOfGPUCallbackHandlers(8) \
        .setNumberOfGPUTaskHandlers(2).setDisplayInterval(100).displayAccumulatedLossValue(True).queueMeasurements(True) \
        .setTaskQueueSizeLimit(32).setPerformanceMonitorInterval(2000).setNumberOfResultSlots(128).allowMemoryReuse(True) \
        .autotuneModels(False).useDirectBuffers(True).setMaxNumberOfMappedPartitions(2).setVariableBufferSize(1 << 20)
    assert (s.number_of_gpu_models, s.number_of_callback_handlers, s.number_of_task_handlers, s.monitor_interval) == (3, 8, 2, 2000)
    assert s.display_accumulated_loss and s.queue_measurements and s.reuse_memory and s.mapped_partitions_window == 2 and s.gpu_devices == [0, 1]
    m = ModelConf.reset().setBatchSize(64).setWpc(4).setSlack(0).setNumberOfSplits(2).setTrainingDataset("train").setValidationDataset("test")
    assert m.splits == 2 and m.getDataset(Phase.TRAIN) == "train" and m.getDataset(Phase.CHECK) == "test"
    assert m.getSolverConf().setCurrentStep(1)._step == 1


def test_operator_conf_reference_method_names():
    """Indexed kernel / stride / padding access, learning-rate multipliers, pool / LRN / ReLU / element-wise helpers under the
    reference's names (kernel/conf/*.java)."""
    from crossbow_b200.conf import BatchNormConf, DataTransformConf, LRNConf, MatFactConf
    c = ConvConf().setNumberOfOutputs(8).setKernelSize(2).setKernel(0, 7).setKernel(1, 1).setStride(0, 1).setStride(1, 1) \
        .setPadding(0, 3).setPadding(1, 0).setNumberOfGroup(1).setWeightsLearningRateMultiplier(2.0)
    assert (c.kernel_height, c.kernel_width, c.getPadding(0), c.getPadding(1), c.numberOfOutputs(), c.numberOfGroups()) == (7, 1, 3, 0, 8, 1)
    assert c.getWeightsLearningRateMultiplier() == 2.0 and c.getBiasLearningRateMultiplier() == 1.0
    p = PoolConf().setKernelSize(3).setStrideSize(2).setGlobal(True)
    assert p.isGlobal() and p.getKernelSize() == 3 and p.getStrideSize() == 2 and p.getPaddingSize() == 0
    assert LRNConf().setSize(7).setKappa(2.0).getSize() == 7 and ReLUConf().setReLUCeiling(6).getReLUCeiling() == 6.0
    e = ElementWiseOpConf()
    assert e.numberOfCoefficients() == 0
    e.resizeCoefficients(2)
    assert e.coefficients == [1.0, 1.0]
    d = DataTransformConf()
    assert not d.subtractMean() and d.setMeanPixelValues(1.0, 2.0, 3.0).hasMeanPixel() and d.subtractMean()
    assert BatchNormConf().setBiasLearningRateMultiplier(0.5).getBiasLearningRateMultiplier() == 0.5
    assert MatFactConf().numberOfLatentVariables() == 10


def test_graph_and_model_accessors_under_reference_names():
    from crossbow_b200.models import build
    spec = build("lenet-caffe", solver_conf=SolverConf())
    m = Model()
    df = Dataflow(spec.train)
    nid = df.init(Shape([8, 1, 28, 28]), Shape([8]), m)
    m.finalise()
    g = df.getSubGraph()
    assert nid == df.totalNumberOfOperators() == g.cardinality() and df.numberOfSubGraphs() == 1 and df.getId() == 0
    assert g.getInputShape().array() == [8, 1, 28, 28] and g.isMostUpstream() and g.getNext() is None and g.getBranchFactor() == 1
    assert g.getDataflowNode() is g.head and g.head.getOrder() == 0 and g.head.getNextList()[0].getPreviousList() == [g.head]
    assert "digraph" in df.exportDot() and "operators" in g.dump() and df.dumpMemoryRequirements()
    w = m.getVariable(0, 1)
    assert m.getSize() == len(m.getVariables()) == 8 and m.capacity() == 4 * m.elements and w.getName() == "weights"
    assert w.getShape().array() == [20, 1, 5, 5] and w.capacity() == 2000 and w.getLearningRateMultiplier() == 1.0 and m.getVariable(99) is None
    s = Shape([2, 3, 4, 5])
    assert s.offset(1, 2) == 100 and s.getNCHW() == [2, 3, 4, 5] and s.countElements(2) == 20 and s.equals(Shape([2, 3, 4, 5])) and s.toString() == "[2, 3, 4, 5]"
    s.push(6)
    assert s.dimensions() == 5
    g2 = SubGraph(DataflowNode(Operator("x", ReLU(ReLUConf()))))
    assert g.connectTo(g2) is g2 and g2.getPrevious() is g and not g2.isMostUpstream()


def _two_halves(joined_by_nodes: bool):
    """LeNet-like network cut after the first pooling layer: (head of the first half, head of the second half)."""
    from crossbow_b200.graph import append_gradients
    from crossbow_b200.models._builder import Net
    from crossbow_b200.types import PoolMethod
    a = Net()
    a.conv("Conv", 8, 5, bias=True)
    a.pool("Pool", PoolMethod.MAX, 2, 2)
    b = Net()
    if joined_by_nodes:
        b.cur = a.cur
    b.conv("Conv", 12, 5, bias=True)
    head_b = b.cur
    b.pool("Pool", PoolMethod.MAX, 2, 2)
    b.fc("InnerProduct", 32)
    b.relu("ReLU")
    b.fc("InnerProduct", 10)
    b.classifier_tail()
    append_gradients(head_b, ModelConf.getInstance().getSolverConf())     # the second half is trained, the first is not
    return a.head, head_b


def test_chained_subgraphs_run_as_one_program():
    """`SubGraph.connectTo`: the output batch of a sub-graph feeds the next one on the same replica
    (dispatcher/TransientTaskDispatcher.java:41-52).  A two-sub-graph dataflow must train exactly like the same operators
    wired into one graph."""
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.data import SyntheticDataset
    from crossbow_b200.graph import SubGraph
    losses = []
    for chained in (True, False):
        SystemConf.reset().setNumberOfCpuModels(2).setDisplayInterval(0)
        mc = ModelConf.reset()
        mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.05).setMomentum(0.9).setAlpha(0.1)
        mc.setBatchSize(8).setWpc(2).setUpdateModel("SMA")
        mc.setDataset(Phase.TRAIN, SyntheticDataset([1, 28, 28], 10, 8, batches=4, seed=2, distribution="uniform"))
        head_a, head_b = _two_halves(joined_by_nodes=not chained)
        if chained:
            first, second = SubGraph(head_a), SubGraph(head_b)
            assert first.connectTo(second) is second and first.getNext() is second and second.getPrevious() is first
            df = Dataflow(first).setPhase(Phase.TRAIN)
            assert df.numberOfSubGraphs() == 2
            joined = df.executable()
            assert joined.numberOfOperators() == first.numberOfOperators() + second.numberOfOperators()
            assert joined.getLossNode() is not None and df.executable() is joined
        else:
            df = Dataflow(SubGraph(head_a)).setPhase(Phase.TRAIN)
        ctx = ExecutionContext([df, None], quiet=True)
        ctx.init()
        ctx.train(8, "tasks")
        losses.append(ctx.measurements.losses())
        ctx.destroy()
    assert len(losses[0]) == 8 and losses[0] == losses[1]
    assert losses[0][-1] < losses[0][0]


def test_debug_checksums_print_one_line_per_operator(tmp_path):
    """`--debug-checksums true`: the CPU engine prints the checksum of every operator's output, as the reference does under
    debug logging (Operator.java:232-259, SubGraph.java:261-262)."""
    from crossbow_b200.context import ExecutionContext
    from crossbow_b200.data import SyntheticDataset
    from crossbow_b200.models import build
    from crossbow_b200.oracle import OracleExecutor
    sysc, mc = SystemConf.reset(), ModelConf.reset()
    sysc.setCPU(True).setGPU(False).setNumberOfCPUModels(1).setDisplayInterval(0)
    sysc.debug_checksums = True
    sc = mc.getSolverConf().setLearningRateDecayPolicy("FIXED").setBaseLearningRate(0.01)
    mc.setBatchSize(4).setWpc(1).setUpdateModel("DEFAULT")
    mc.setDataset(Phase.TRAIN, SyntheticDataset([1, 28, 28], 10, 4, batches=2, seed=1))
    spec = build("lenet-caffe", solver_conf=sc)
    ctx = ExecutionContext([Dataflow(spec.train).setPhase(Phase.TRAIN), None], quiet=True)
    lines = []
    ctx.emit = lines.append
    ctx.init()
    try:
        ctx.train(1, "tasks")
    finally:
        ctx.destroy()
    assert OracleExecutor.checksum_sink is None                      # switched off again with the context
    sums = [l for l in lines if l.startswith("Kernel's ")]
    names = [l.split("'s ")[1].split(" output")[0] for l in sums]
    assert names[:3] == ["Conv", "Pool", "Conv"] and "SoftMaxLossGradient" in names and names[-1] == "ConvGradient"
    soft = next(l for l in sums if "SoftMax output" in l)
    assert soft.endswith("is 4.00000")                               # four rows of probabilities


def test_measurement_log_parser_matches_the_reference_tool(tmp_path):
    """tools/measurements/parse-measurements.py: percentiles of GPU and memory utilisation per device from an nvidia-smi
    CSV log, optionally between two moments; idle devices stay out of the aggregate."""
    from datetime import datetime
    from crossbow_b200.utils import gpumon
    assert gpumon.sampler_command(200)[:2] == ["nvidia-smi", "--query-gpu=timestamp,gpu_serial,temperature.gpu,utilization.gpu,utilization.memory,memory.used,memory.free"]
    p = tmp_path / "measurements.csv"
    rows = ["# Thu Jan  1 00:00:00 UTC 2026", "timestamp, gpu_serial, temperature.gpu, utilization.gpu, utilization.memory, memory.used, memory.free"]
    for i in range(100):
        ts = f"2026/01/01 00:00:{i // 5:02d}.{(i % 5) * 200:03d}"
        rows.append(f"{ts}, A1, 50, {i}, {i / 2}, 1000, 179000")
        rows.append(f"{ts}, B2, 40, 0, 0, 10, 180000")                  # an idle device
    p.write_text("\n".join(rows) + "\n")
    st = gpumon.parse_measurements(str(p))
    assert st["A1"]["samples"] == 100 and st["B2"]["samples"] == 100
    g = st["A1"]["gpu_util"]
    assert g["min"] == 0 and g["max"] == 99 and abs(g["mean"] - 49.5) < 1e-9 and abs(g["p50"] - 49.5) < 1e-9 and abs(g["p99"] - 98.01) < 1e-6
    assert abs(st["A1"]["mem_util"]["p25"] - 12.375) < 1e-9
    assert st["all"]["samples"] == 100                                   # the idle device is left out of the aggregate
    t0 = int(datetime.strptime("2026/01/01 00:00:10.000", "%Y/%m/%d %H:%M:%S.%f").timestamp() * 1000)
    half = gpumon.parse_measurements(str(p), start_ms=t0)
    assert half["A1"]["samples"] == 50 and half["A1"]["gpu_util"]["min"] == 50
    assert gpumon.main(["parse", str(p)]) == 0
